"""The operator language: typed expression nodes, the per-trace builder and the user-visible DSL functions.

Calling an operator function under a :class:`TraceBuilder` records every DSL operation as a :class:`Node`
appended, in program order, to the innermost open :class:`Block`.  Loops and conditionals own nested blocks
(structured regions) instead of the reference's flat BEGIN/END marker expressions
(opveclib/expression.py:1964-2183); everything else carries the same information as the reference's
``Expression`` messages (opveclib/language.proto:374-404) and follows the same typing rules:

* python ``int`` -> int64 constant, python ``float`` -> float64 constant, then cast to the other operand's
  dtype; two python constants are an error (opveclib/expression.py:1132-1141, 1702-1716);
* both operands of a binary operation have the same dtype, which is also the result's dtype - comparisons and
  logicals included (opveclib/expression.py:1718-1730);
* N-d tensor indices are turned into row-major linear offsets computed in uint64, after the user's own index
  arithmetic ran in its own (usually uint32) type (opveclib/expression.py:859-973).

Every value node is evaluated where it was traced, so a read of a variable sees the value assigned so far.
"""
import threading

import numpy as np

from .dtypes import (DType, TensorType, _is_int, float32, float64, int8, int16, int32, int64, uint8, uint16,
                     uint32, uint64)

# ---------------------------------------------------------------------------------------------------------
# operation tables: which dtypes each math node accepts (opveclib/expression.py:1430-1456, 1632-1672)
_F = (float32.code, float64.code)
_SIGNED = _F + (int8.code, int16.code, int32.code, int64.code)
_ALL = _SIGNED + (uint8.code, uint16.code, uint32.code, uint64.code)
_ALL_WITH_HALF = (1,) + _ALL

UNARY_DOMAIN = {
    'acos': _F, 'asin': _F, 'atan': _F, 'cos': _F, 'cosh': _F, 'sin': _F, 'sinh': _F, 'tan': _F, 'tanh': _F,
    'exp': _F, 'log': _F, 'log10': _F, 'sqrt': _F, 'ceil': _F, 'floor': _F,
    'abs': _F + (int8.code, int16.code, int32.code, int64.code),
    'negate': _SIGNED, 'not': _ALL, 'isinf': _F, 'isfinite': _F, 'isnan': _F,
}
BINARY_DOMAIN = {
    'add': _ALL_WITH_HALF, 'sub': _ALL_WITH_HALF, 'mul': _ALL_WITH_HALF, 'div': _ALL_WITH_HALF,
    'mod': _ALL_WITH_HALF, 'eq': _ALL_WITH_HALF, 'ne': _ALL_WITH_HALF, 'lt': _ALL_WITH_HALF,
    'le': _ALL_WITH_HALF, 'gt': _ALL_WITH_HALF, 'ge': _ALL_WITH_HALF, 'min': _ALL_WITH_HALF,
    'max': _ALL_WITH_HALF, 'and': _ALL_WITH_HALF, 'or': _ALL_WITH_HALF, 'pow': _F, 'atan2': _F,
}
LIMIT_KINDS = ('min_value', 'max_value', 'epsilon')


# ---------------------------------------------------------------------------------------------------------
class Block(object):
    """An ordered list of nodes: the body of an operator, of a loop or of one branch of a conditional."""
    __slots__ = ('nodes',)

    def __init__(self):
        self.nodes = []


class Node(object):
    """Base of every traced expression.  ``kind`` names the node class in serialised form, ``args`` are the
    operand nodes, ``attr`` holds compile-time data."""
    kind = None
    is_scalar = False
    is_tensor = False

    def __init__(self):
        self.args = []
        self.attr = {}

    def _register(self):
        _builder().emit(self)
        return self

    def __bool__(self):
        raise SyntaxError('Attempting to interpret the truth of an expression. This typically happens when '
                          'trying to use a python native "if", "min", or "max" statement to create a '
                          'data-dependent conditional inside of an operator, which is not supported. To do so '
                          'you must use the corresponding "with if_(...)", "minimum", and "maximum" '
                          'functions.')

    def __ilshift__(self, other):
        raise SyntaxError('Can only use assignment operator <<= on a variable.')

    __hash__ = object.__hash__


class Scalar(Node):
    """A single typed value."""
    is_scalar = True

    def __init__(self, dtype):
        if not isinstance(dtype, DType):
            raise TypeError('Scalar expressions must be initialized with a DType')
        super(Scalar, self).__init__()
        self.dtype = dtype

    def __add__(self, other):
        return _binary('add', self, other)

    def __radd__(self, other):
        return _binary('add', other, self)

    def __sub__(self, other):
        return _binary('sub', self, other)

    def __rsub__(self, other):
        return _binary('sub', other, self)

    def __mul__(self, other):
        return _binary('mul', self, other)

    def __rmul__(self, other):
        return _binary('mul', other, self)

    def __truediv__(self, other):
        return _binary('div', self, other)

    def __rtruediv__(self, other):
        return _binary('div', other, self)

    __div__ = __truediv__
    __rdiv__ = __rtruediv__

    def __mod__(self, other):
        return _binary('mod', self, other)

    def __rmod__(self, other):
        return _binary('mod', other, self)

    def __eq__(self, other):
        return _binary('eq', self, other)

    def __ne__(self, other):
        return _binary('ne', self, other)

    def __lt__(self, other):
        return _binary('lt', self, other)

    def __le__(self, other):
        return _binary('le', self, other)

    def __gt__(self, other):
        return _binary('gt', self, other)

    def __ge__(self, other):
        return _binary('ge', self, other)

    def __neg__(self):
        return _unary('negate', self)

    __hash__ = object.__hash__


class TensorExpr(Node):
    """A node that denotes a whole tensor (input, output, position, constant or worker-local array)."""
    is_tensor = True
    readable = False
    writable = False

    def __init__(self, tensor_type):
        super(TensorExpr, self).__init__()
        self.tensor_type = tensor_type
        self.dtype = tensor_type.dtype
        self.shape = tensor_type.shape
        self.size = tensor_type.size
        self.rank = tensor_type.rank

    def __getitem__(self, item):
        if not self.readable:
            raise TypeError('Can only index a readable tensor.')
        return ReadTensor(self, _to_scalar_index(self.shape, item))

    def __setitem__(self, key, value):
        if not self.writable:
            raise TypeError('Can only assign to writable tensors.')
        AssignTensor(self, _to_scalar_index(self.shape, key), value)


# ---------------------------------------------------------------------------------------------------------
class InputTensor(TensorExpr):
    kind = 'input'
    readable = True

    def __init__(self, tensor_type, io_index):
        if not isinstance(tensor_type, TensorType):
            raise TypeError
        if not _is_int(io_index):
            raise TypeError
        if io_index < 0 or io_index > 2 ** 32 - 1:
            raise ValueError
        super(InputTensor, self).__init__(tensor_type)
        self.attr['io_index'] = int(io_index)
        self._register()


class OutputTensor(TensorExpr):
    kind = 'output'
    writable = True

    def __init__(self, tensor_type, io_index):
        if not isinstance(tensor_type, TensorType):
            raise TypeError
        if not _is_int(io_index):
            raise TypeError
        if io_index < 0 or io_index > 2 ** 32 - 1:
            raise ValueError
        super(OutputTensor, self).__init__(tensor_type)
        self.attr['io_index'] = int(io_index)
        self._register()


class PositionTensor(TensorExpr):
    """The worker's coordinates in the workgroup: a uint32 vector with one entry per workgroup dimension."""
    kind = 'position'
    readable = True

    def __init__(self, workgroup_shape):
        if _is_int(workgroup_shape):
            shape = [int(workgroup_shape)]
        else:
            try:
                shape = []
                for elem in workgroup_shape:
                    if not _is_int(elem):
                        raise TypeError
                    shape.append(int(elem))
            except TypeError:
                raise TypeError('workgroup_shape must be an int or an iterable of ints')
        super(PositionTensor, self).__init__(TensorType([len(shape)], uint32))
        self.workgroup_shape = shape
        self.attr['workgroup_shape'] = list(shape)
        self._register()


class ConstScalar(Scalar):
    """A python number: int -> int64, float -> float64."""
    kind = 'const'

    def __init__(self, value):
        if isinstance(value, (bool, np.bool_)):
            raise TypeError('Tried to wrap a bool as a ConstScalar. Can only wrap an int or float')
        if isinstance(value, (float, np.floating)):
            super(ConstScalar, self).__init__(float64)
            self.attr['value'] = float(value)
        elif _is_int(value):
            super(ConstScalar, self).__init__(int64)
            self.attr['value'] = int(value)
        else:
            raise TypeError('Tried to wrap a ' + str(type(value)) + ' as a ConstScalar. Can only wrap an int '
                            'or float')
        self._register()

    def value(self):
        return self.attr['value']


class ConstTensor(TensorExpr):
    kind = 'const_tensor'
    readable = True

    def __init__(self, value):
        if isinstance(value, (list, tuple)):
            array = np.array(value)
        elif isinstance(value, np.ndarray):
            array = value
        elif _is_int(value) or isinstance(value, float):
            array = np.array([value])
        else:
            raise TypeError('ConstTensors can wrap lists, tuples, and numpy arrays')
        if array.dtype == np.object_ or array.dtype.kind not in 'fiu':
            raise TypeError('ConstTensors can wrap lists, tuples, and numpy arrays of numbers')
        super(ConstTensor, self).__init__(TensorType.like(array))
        self.attr['data'] = np.ascontiguousarray(array).reshape(-1).tolist()
        self._register()

    def to_array(self):
        return np.array(self.attr['data'], dtype=self.dtype.as_numpy())


class Variable(Scalar):
    """A worker-local mutable scalar; assigned with ``<<=``."""
    kind = 'variable'

    def __init__(self, dtype, initial_const):
        if not isinstance(initial_const, ConstScalar):
            raise TypeError('Variables must be initialized with a constant scalar')
        if not isinstance(dtype, DType):
            raise TypeError('dtype must be a DType')
        super(Variable, self).__init__(dtype)
        self.args = [initial_const]
        self._register()

    def __ilshift__(self, other):
        AssignVariable(self, other)
        return self

    __hash__ = object.__hash__


class Cast(Scalar):
    kind = 'cast'

    def __init__(self, dtype, target):
        if not isinstance(dtype, DType):
            raise TypeError('dtype must be a DType')
        if not isinstance(target, Scalar):
            raise TypeError('Can only cast scalar expressions. Received ' + str(type(target)) + ': ' +
                            str(target))
        super(Cast, self).__init__(dtype)
        self.args = [target]
        self._register()


class AssignVariable(Node):
    kind = 'assign_var'

    def __init__(self, scalar_expr, value_expr):
        if not isinstance(scalar_expr, Variable):
            raise TypeError('Can only assign to a variable')
        if isinstance(value_expr, Scalar):
            value = value_expr
        else:
            value = Cast(scalar_expr.dtype, ConstScalar(value_expr))
        if value.dtype != scalar_expr.dtype:
            raise TypeError('cannot assign ' + str(value.dtype) + ' to ' + str(scalar_expr.dtype) + ' scalar')
        super(AssignVariable, self).__init__()
        self.args = [scalar_expr, value]
        self._register()


class UnaryMath(Scalar):
    kind = 'unary'

    def __init__(self, fn, arg):
        if fn not in UNARY_DOMAIN:
            raise ValueError(str(fn) + ' is an invalid unary math code.')
        if not isinstance(arg, Scalar):
            raise TypeError('Must apply math functions to scalar expressions. Received: ' + str(arg))
        if arg.dtype.code not in UNARY_DOMAIN[fn]:
            raise ValueError(str(arg.dtype) + ' arguments not supported for unary math function ' + fn.upper())
        super(UnaryMath, self).__init__(arg.dtype)
        self.attr['fn'] = fn
        self.args = [arg]
        self._register()


class Limit(Scalar):
    kind = 'limit'

    def __init__(self, which, dtype):
        if which not in LIMIT_KINDS:
            raise ValueError(str(which) + ' is an invalid limits code.')
        if not isinstance(dtype, DType):
            raise TypeError('Must apply limits functions to dtypes. Received: ' + str(dtype))
        if dtype.code not in _F:
            raise ValueError(str(dtype) + ' arguments not supported for limits function ' + which.upper())
        super(Limit, self).__init__(dtype)
        self.attr['which'] = which
        self._register()


class BinaryMath(Scalar):
    kind = 'binary'

    def __init__(self, fn, arg1, arg2):
        if fn not in BINARY_DOMAIN:
            raise ValueError('Invalid binary math code')
        a = _wrap_const(arg1)
        b = _wrap_const(arg2)
        if not isinstance(a, Node):
            raise TypeError('Cannot apply ' + fn.upper() + ' to first non-expression argument:\n' + str(a))
        if not isinstance(b, Node):
            raise TypeError('Cannot apply ' + fn.upper() + ' to second non-expression argument:\n' + str(b))
        if not isinstance(a, Scalar):
            raise TypeError('First argument to ' + fn.upper() + ' must be a scalar expression, got:\n' + str(a))
        if not isinstance(b, Scalar):
            raise TypeError('Second argument to ' + fn.upper() + ' must be a scalar expression, got:\n' + str(b))
        a_const = type(a) is ConstScalar
        b_const = type(b) is ConstScalar
        if a_const and b_const:
            raise TypeError('Cannot apply binary operator to two constants.')
        if b_const:
            b = Cast(a.dtype, b)
        elif a_const:
            a = Cast(b.dtype, a)
        if a.dtype != b.dtype:
            raise TypeError('arg1 type (' + str(a.dtype) + ') must be the same as arg2 type (' + str(b.dtype) +
                            ')')
        if a.dtype.code not in BINARY_DOMAIN[fn]:
            raise ValueError(str(a.dtype) + ' arguments not supported for binary math function ' + fn.upper())
        super(BinaryMath, self).__init__(a.dtype)
        self.attr['fn'] = fn
        self.args = [a, b]
        self._register()


class LocalTensor(TensorExpr):
    """A worker-local array initialised from a constant tensor."""
    kind = 'local'
    readable = True
    writable = True

    def __init__(self, initial_value):
        if type(initial_value) is not ConstTensor:
            raise TypeError('Tensors must be initialized by ConstTensors')
        super(LocalTensor, self).__init__(initial_value.tensor_type)
        self.args = [initial_value]
        self._register()


class AssignTensor(Node):
    kind = 'assign_tensor'

    def __init__(self, tensor_expr, index_expr, value_expr):
        if not (isinstance(tensor_expr, TensorExpr) and tensor_expr.writable):
            raise TypeError('Can only assign to writable tensors.')
        index = _check_index(tensor_expr, index_expr)
        if isinstance(value_expr, Node):
            value = value_expr
        else:
            value = Cast(tensor_expr.dtype, ConstScalar(value_expr))
        if not isinstance(value, Scalar) or value.dtype != tensor_expr.dtype:
            got = str(value.dtype) if isinstance(value, Scalar) else str(type(value))
            raise TypeError('cannot assign ' + got + ' to ' + str(tensor_expr.dtype) + ' tensor')
        super(AssignTensor, self).__init__()
        self.args = [tensor_expr, index, value]
        self._register()


class ReadTensor(Scalar):
    kind = 'read'

    def __init__(self, tensor_expr, index_expr):
        if not (isinstance(tensor_expr, TensorExpr) and tensor_expr.readable):
            raise TypeError('Can only index a readable tensor.')
        index = _check_index(tensor_expr, index_expr)
        super(ReadTensor, self).__init__(tensor_expr.dtype)
        self.args = [tensor_expr, index]
        self._register()


class ForRange(Node):
    """``for (var = start; (var < stop && step > 0) || (var > stop && step < 0); var += step) body``
    (opveclib/expression.py:1996-2006)."""
    kind = 'for'

    def __init__(self, index, start, stop, step):
        for e in (start, stop, step):
            if e.dtype != index.dtype:
                raise TypeError('All input expressions must have the same type.')
        super(ForRange, self).__init__()
        self.args = [index, start, stop, step]
        self.body = Block()
        self._state = 0
        self._register()

    def __iter__(self):
        return self

    def __next__(self):
        if self._state == 0:
            self._state = 1
            _builder().push(self.body)
            return self.args[0]
        if self._state == 1:
            self._state = 2
            _builder().pop(self.body)
        raise StopIteration

    next = __next__


class IfChain(Node):
    """``if (c0) b0 else if (c1) b1 ... else bn``.  ``conds[i]`` is None for the trailing else branch.  The
    nodes that compute an elif condition sit in the enclosing block *before* the chain, as the reference hoists
    them (opveclib/expression.py:374-439)."""
    kind = 'if'

    def __init__(self, condition):
        super(IfChain, self).__init__()
        self.conds = [condition]
        self.blocks = [Block()]
        self.args = [condition]
        self._register()

    def add_branch(self, condition):
        if self.conds[-1] is None:
            raise SyntaxError('Could not find prior if block')
        self.conds.append(condition)
        self.blocks.append(Block())
        if condition is not None:
            self.args.append(condition)


class _Branch(object):
    """Context manager returned by if_/elif_/else_."""

    def __init__(self, kind, condition):
        if kind != 'else':
            if not isinstance(condition, Scalar):
                if isinstance(condition, bool):
                    raise TypeError('Attempting to use a constant boolean, %s, with the operator if_ '
                                    'expression. Use the python if instead since this can be interpreted at '
                                    'operator definition time.' % condition)
                raise TypeError('Condition must be a scalar expression, instead got: ' + str(condition))
        self.kind = kind
        self.condition = condition
        self.block = None
        if kind == 'if':
            self.chain = IfChain(condition)
        else:
            self.chain = None

    def __enter__(self):
        b = _builder()
        if self.kind == 'if':
            self.block = self.chain.blocks[0]
        else:
            self.chain = b.reopen_chain()
            self.chain.add_branch(self.condition)
            self.block = self.chain.blocks[-1]
        b.push(self.block)

    def __exit__(self, exc_type, exc_val, exc_tb):
        _builder().pop(self.block)
        return False


# ---------------------------------------------------------------------------------------------------------
class TraceBuilder(object):
    """Collects the nodes of one operator trace.  One builder per traced call; the active builder is held in
    thread-local storage for the duration of the call only."""

    def __init__(self):
        self.root = Block()
        self.stack = [self.root]
        self.inputs = []
        self.outputs = []
        self.position = None
        self.count = 0

    def emit(self, node):
        if isinstance(node, PositionTensor):
            if self.position is not None:
                raise ValueError('Already defined the position tensor.')
            self.position = node
        elif isinstance(node, OutputTensor):
            if node.attr['io_index'] != len(self.outputs):
                raise ValueError('Trying to add outputs to expression dag out of order')
            self.outputs.append(node)
        elif isinstance(node, InputTensor):
            if node.attr['io_index'] != len(self.inputs):
                raise ValueError('Trying to add inputs to expression dag out of order')
            self.inputs.append(node)
        node.uid = self.count
        self.count += 1
        self.stack[-1].nodes.append(node)

    def push(self, block):
        self.stack.append(block)

    def pop(self, block):
        if self.stack[-1] is not block:
            raise SyntaxError('Unbalanced control flow blocks')
        self.stack.pop()

    def reopen_chain(self):
        """Find the conditional an elif_/else_ continues: the last IfChain of the current block.  Whatever was
        traced after it (the elif condition's operands) is moved in front of it."""
        nodes = self.stack[-1].nodes
        for i in range(len(nodes) - 1, -1, -1):
            if isinstance(nodes[i], IfChain):
                chain = nodes[i]
                trailing = nodes[i + 1:]
                del nodes[i:]
                nodes.extend(trailing)
                nodes.append(chain)
                return chain
        raise SyntaxError('Could not find prior if block')


_tls = threading.local()


def _builder():
    b = getattr(_tls, 'builder', None)
    if b is None:
        raise RuntimeError('Expressions can only be created while an operator function is being traced.')
    return b


class tracing(object):
    """``with tracing() as builder:`` activates a fresh builder for the calling thread."""

    def __enter__(self):
        self.prev = getattr(_tls, 'builder', None)
        self.builder = TraceBuilder()
        _tls.builder = self.builder
        return self.builder

    def __exit__(self, exc_type, exc_val, exc_tb):
        _tls.builder = self.prev
        return False


# ---------------------------------------------------------------------------------------------------------
def _wrap_const(x):
    if isinstance(x, Node):
        return x
    try:
        return ConstScalar(x)
    except TypeError:
        return x


def _binary(fn, a, b):
    return BinaryMath(fn, a, b)


def _unary(fn, a):
    return UnaryMath(fn, a)


def _check_index(target_expr, index_expr):
    if isinstance(index_expr, Node):
        index = index_expr
    else:
        index = ConstScalar(index_expr)
    if not isinstance(index, Scalar):
        raise TypeError('Can only index with a scalar.')
    if type(index) is ConstScalar:
        if target_expr.size <= index.value() or index.value() < 0:
            raise IndexError('Index out of bounds.')
    return index


def _to_scalar_index(target_shape, index):
    """N-d index -> row-major linear offset.  Accepts a 1-D index tensor (position, input, local or constant)
    with one entry per dimension, a scalar expression for rank-1 targets, or a list/tuple mixing python ints,
    scalar expressions and size-1 tensors; constant entries are bounds-checked at trace time
    (opveclib/expression.py:859-973)."""
    target_rank = len(target_shape)
    block_size = [1]
    for cur_dim in range(target_rank - 1, 0, -1):
        block_size.append(block_size[-1] * target_shape[cur_dim])
    block_size.reverse()

    index_expr = index
    if not isinstance(index, Node):
        try:
            index_expr = ConstTensor(index)
        except TypeError:
            index_expr = index

    if isinstance(index_expr, Scalar):
        index_expr = [index_expr]

    if isinstance(index_expr, (list, tuple)):
        if target_rank != len(index_expr):
            raise IndexError('length of index list (' + str(len(index_expr)) +
                             ') must match indexed tensor rank (' + str(target_rank) + ')')
        entries = []
        for value in index_expr:
            if isinstance(value, Node):
                if not isinstance(value, Scalar):
                    if isinstance(value, TensorExpr) and value.size == 1:
                        value = value[0]
                    else:
                        raise TypeError('Must index tensors with an int or a scalar expression. Instead '
                                        'got:\n' + str(value))
                entries.append(value)
            else:
                cur_shape = target_shape[len(entries)]
                cur_value = int(np.floor(value))
                if cur_value >= cur_shape or cur_value < 0:
                    raise IndexError('Expected index to be in range [0, ' + str(cur_shape) +
                                     '), but received index value ' + str(cur_value))
                entries.append(cur_value)
        result = None
        for i, entry in enumerate(entries):
            bound = entry if _is_int(entry) else Cast(uint64, entry)
            term = bound * block_size[i]
            result = term if result is None else result + term
        return result

    if type(index_expr) is ConstTensor:
        if len(index_expr.shape) != 1:
            raise IndexError('Index must be one dimensional')
        if index_expr.shape[0] != target_rank:
            raise IndexError('length of index tensor (' + str(index_expr.shape[0]) +
                             ') must match indexed tensor rank (' + str(target_rank) + ')')
        data = np.floor(index_expr.to_array())
        result = 0
        for i, elem in enumerate(data):
            cur_value = int(elem)
            if cur_value >= target_shape[i] or cur_value < 0:
                raise IndexError('Expected index to be in range [0, ' + str(target_shape[i]) +
                                 '), but received index value ' + str(cur_value))
            result += cur_value * block_size[i]
        return result

    if type(index_expr) in (LocalTensor, PositionTensor, InputTensor):
        if len(index_expr.shape) != 1:
            raise IndexError('Index must be one dimensional')
        if index_expr.shape[0] != target_rank:
            raise IndexError('length of index tensor (' + str(index_expr.shape[0]) +
                             ') must match indexed tensor rank (' + str(target_rank) + ')')
        result = None
        for i in range(target_rank):
            term = Cast(uint64, ReadTensor(index_expr, i)) * block_size[i]
            result = term if result is None else result + term
        return result

    raise TypeError('Cannot index a tensor with a ' + str(type(index_expr)))


def _tensor_type_polymorphic(*args):
    err_msg = 'Expected a TensorType or a shape and a dtype as arguments'
    if len(args) == 1:
        if type(args[0]) is not TensorType:
            raise TypeError(err_msg)
        return args[0]
    if len(args) == 2:
        return TensorType(args[0], args[1])
    raise TypeError(err_msg)


# ---------------------------------------------------------------------------------------------------------
# user-visible DSL functions (names as exported by the reference, opveclib/__init__.py:11-48)
def input(*args):
    """Declare the next input tensor of the operator being traced."""
    return InputTensor(_tensor_type_polymorphic(*args), len(_builder().inputs))


def output(*args):
    """Declare a new output tensor from a TensorType, or from a shape and a dtype."""
    return OutputTensor(_tensor_type_polymorphic(*args), len(_builder().outputs))


def output_like(other):
    """Declare a new output tensor with the TensorType of another tensor."""
    return output(TensorType.like(other))


def position_in(workgroup_shape):
    """Define the workgroup shape (once per operator) and get the worker's position in it."""
    return PositionTensor(workgroup_shape)


def variable(initial_value, dtype):
    """Declare a worker-local variable.  A python number initialises it directly; a scalar expression is
    assigned to a zero-initialised variable (opveclib/expression.py:1309-1324)."""
    if _is_int(initial_value) or isinstance(initial_value, float):
        return Variable(dtype, ConstScalar(initial_value))
    if isinstance(initial_value, Scalar):
        var = Variable(dtype, ConstScalar(0))
        var <<= initial_value
        return var
    raise TypeError('Must initialize a variable with a numeric constant or a scalar expression.')


def cast(value, dtype):
    return Cast(dtype, value)


def zeros(shape, dtype):
    """A worker-local tensor initialised to zero."""
    return LocalTensor(ConstTensor(np.zeros(shape, dtype=DType(dtype).as_numpy())))


def ones(shape, dtype):
    """A worker-local tensor initialised to one."""
    return LocalTensor(ConstTensor(np.ones(shape, dtype=DType(dtype).as_numpy())))


def min_value(dtype):
    """Smallest positive normal value of a floating point dtype."""
    return Limit('min_value', dtype)


def max_value(dtype):
    return Limit('max_value', dtype)


def epsilon(dtype):
    return Limit('epsilon', dtype)


def arccos(x):
    return _unary('acos', x)


def arcsin(x):
    return _unary('asin', x)


def arctan(x):
    return _unary('atan', x)


def cos(x):
    return _unary('cos', x)


def cosh(x):
    return _unary('cosh', x)


def sin(x):
    return _unary('sin', x)


def sinh(x):
    return _unary('sinh', x)


def tan(x):
    return _unary('tan', x)


def tanh(x):
    return _unary('tanh', x)


def exp(x):
    return _unary('exp', x)


def log(x):
    return _unary('log', x)


def log10(x):
    return _unary('log10', x)


def sqrt(x):
    return _unary('sqrt', x)


def ceil(x):
    return _unary('ceil', x)


def floor(x):
    return _unary('floor', x)


def absolute(x):
    return _unary('abs', x)


def logical_not(x):
    return _unary('not', x)


def isinf(x):
    return _unary('isinf', x)


def isfinite(x):
    return _unary('isfinite', x)


def isnan(x):
    return _unary('isnan', x)


def minimum(x, y):
    return _binary('min', x, y)


def maximum(x, y):
    return _binary('max', x, y)


def power(x, y):
    return _binary('pow', x, y)


def arctan2(x, y):
    return _binary('atan2', x, y)


def logical_and(x, y):
    return _binary('and', x, y)


def logical_or(x, y):
    return _binary('or', x, y)


def arange(start, stop=None, step=None):
    """``for i in arange(...)``: a counted loop inside the operator.  The loop variable takes the dtype of the
    first expression among (start, stop, step), else int64 (opveclib/expression.py:1908-1961)."""
    if stop is None:
        start_inferred, stop_inferred = 0, start
    else:
        start_inferred, stop_inferred = start, stop
    step_inferred = 1 if step is None else step

    operands = []
    first_type = None
    for val in (start_inferred, stop_inferred, step_inferred):
        if isinstance(val, Node):
            operands.append(val)
            if first_type is None:
                first_type = val.dtype
        else:
            operands.append(ConstScalar(val))
    if first_type is None:
        first_type = int64 if _is_int(start) else float64
    casted = [Cast(first_type, e) if type(e) is ConstScalar else e for e in operands]
    index = variable(0, first_type)
    return ForRange(index, casted[0], casted[1], casted[2])


def if_(condition):
    """``with if_(cond):`` - data dependent conditional execution."""
    return _Branch('if', condition)


def elif_(condition):
    """``with elif_(cond):`` - must directly follow an if_ or elif_ block."""
    return _Branch('elif', condition)


def else_():
    """``with else_():`` - must directly follow an if_ or elif_ block."""
    return _Branch('else', None)
