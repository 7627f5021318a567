"""Operator definition and the lazy operator graph.

``@operator()`` turns a python function written in the DSL into an operator generator; calling it traces the
function for the argument types into a :class:`~opveclib_b200.kernel.KernelIR` and returns a lazy
:class:`Operator` node whose inputs are arrays or the outputs of other operators.  ``@gradient(op)`` attaches a
user-defined gradient, traced into its own operator graph at call time.  Behaviour follows
opveclib/operator.py:134-673 (definition) and 679-806 (graph construction).
"""
import dis
import inspect

import numpy as np

from .dtypes import TensorType
from .kernel import trace_function
from .local import logger


# Infix operators of lazy operator results: python method name -> (key of the operator library entry, whether the
# lazy value is the right-hand operand).  The library (stdops) registers its element-wise operators under these
# keys; the methods are attached to both classes below.
_INFIX = {
    '__add__': ('add', False), '__radd__': ('add', True), '__sub__': ('sub', False), '__rsub__': ('sub', True),
    '__mul__': ('mul', False), '__rmul__': ('mul', True), '__truediv__': ('div', False),
    '__rtruediv__': ('div', True), '__div__': ('div', False), '__rdiv__': ('div', True),
    '__mod__': ('mod', False), '__rmod__': ('mod', True), '__eq__': ('eq', False), '__ne__': ('ne', False),
    '__lt__': ('lt', False), '__le__': ('le', False), '__gt__': ('gt', False), '__ge__': ('ge', False),
}
_infix_library = {}


def _attach_infix(cls, unwrap):
    """Give ``cls`` the infix methods; ``unwrap(self)`` yields the OperatorOutput that takes part."""
    def binary(key, reflected):
        def method(self, other):
            mine = unwrap(self)
            fn = _infix_library[key]
            return fn(other, mine) if reflected else fn(mine, other)
        return method

    for method_name, (key, reflected) in _INFIX.items():
        setattr(cls, method_name, binary(key, reflected))
    cls.__neg__ = lambda self: _infix_library['neg'](unwrap(self))
    cls.__hash__ = object.__hash__


class OperatorOutput(object):
    """One un-evaluated output tensor of an :class:`Operator` (opveclib/operator.py:134-160).  Arithmetic and
    comparisons between outputs build further operators from the standard operator library."""
    __array_priority__ = 1

    @staticmethod
    def register_magic_method(key, value):
        """Install the library operator behind an infix key ('add', 'lt', 'neg', ...)."""
        _infix_library[key] = value

    def __init__(self, parent, index):
        if not isinstance(parent, Operator) or not isinstance(index, int):
            raise TypeError('an OperatorOutput is (Operator, int output index)')
        self.parent, self.index = parent, index
        t = self.tensor_type = parent.output_types[index]
        self.shape, self.dtype, self.size, self.rank = t.shape, t.dtype, t.size, t.rank

    @property
    def from_gradient(self):
        return self.parent.from_gradient

    def __bool__(self):
        raise SyntaxError('The value of an operator output is not known while the graph is being built.')


_attach_infix(OperatorOutput, lambda out: out)


class GradientPlaceholder(object):
    """Stands for an operator input or an output gradient while a gradient function is traced."""

    def __init__(self, shape, dtype):
        self.tensor_type = TensorType(shape, dtype)
        self.rank = self.tensor_type.rank
        self.shape = list(shape)
        self.dtype = self.tensor_type.dtype
        self.size = self.tensor_type.size


class Operator(object):
    """A lazily evaluated operator application: a traced kernel plus where its inputs come from.  Where a tensor
    is expected (infix arithmetic, ``shape``, ``dtype``) an operator with exactly one output stands for that
    output; one with several must be indexed (SyntaxError otherwise, as in opveclib/operator.py:210-216)."""
    __array_priority__ = 1

    def __init__(self, kernel, inputs, grad_dag, from_gradient, name, generator=None, constants=None):
        self.generator = generator      # the OpGenerator and constants that produced this application, so the
        self.constants = constants      # same operator can be traced again for another input shape
        self.kernel = kernel
        self.inputs = inputs
        self.output_types = kernel.output_types
        self.name = name
        self.grad_dag = grad_dag
        self.from_gradient = from_gradient
        logger.debug('Operator created: ' + str(name))

    def __getitem__(self, item):
        return OperatorOutput(self, item)

    def __len__(self):
        return len(self.output_types)

    def __iter__(self):
        return (OperatorOutput(self, i) for i in range(len(self.output_types)))

    def only_output(self):
        if len(self.output_types) != 1:
            raise SyntaxError(str(self.name) + ' has ' + str(len(self.output_types)) + ' outputs: index the one '
                              'that is meant before using it as a tensor.')
        return self[0]

    @property
    def shape(self):
        return self.only_output().shape

    @property
    def dtype(self):
        return self.only_output().dtype


_attach_infix(Operator, Operator.only_output)


def _resolve_output(x):
    """OperatorOutput of ``x``; single-output Operators resolve to their only output."""
    if isinstance(x, Operator):
        if len(x.output_types) != 1:
            raise ValueError('Only a single-output Operator can be used as an input to another operator. '
                             'Index a specific output from multi-output Operators.')
        return x[0]
    if not isinstance(x, OperatorOutput):
        raise TypeError('Only operator outputs can be used to build an op dag. Received a ' + str(type(x)))
    return x


class OpGenerator(object):
    """The callable an ``@operator()`` decoration returns."""

    def __init__(self, op_function, forbid_none_valued_constants, name):
        self.op_function = op_function
        self.forbid_none_valued_constants = forbid_none_valued_constants
        self.name = op_function.__name__ if name is None else name
        self.grad_function = None
        self.__name__ = op_function.__name__
        self.__doc__ = op_function.__doc__

    def __str__(self):
        return self.op_function.__name__

    def _parameters(self):
        """(names of the tensor parameters, {constant name: default}, accepts *args)."""
        tensors, constants, variadic = [], {}, False
        for p in inspect.signature(self.op_function).parameters.values():
            if p.kind == p.VAR_POSITIONAL:
                variadic = True
            elif p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD):
                if p.default is p.empty:
                    tensors.append(p.name)
                else:
                    constants[p.name] = p.default
            elif p.kind == p.KEYWORD_ONLY and p.default is not p.empty:
                constants[p.name] = p.default
        return tensors, constants, variadic

    def _tensor_arguments(self, inputs):
        """The positional arguments as graph inputs with their tensor types; anything without shape and dtype is
        a TypeError that names the position."""
        resolved, types = [], []
        for position, arg in enumerate(inputs, 1):
            if isinstance(arg, Operator):
                arg = _resolve_output(arg)          # (ValueError for an operator with several outputs)
            try:
                types.append(TensorType.like(arg))
            except (AttributeError, TypeError):
                raise TypeError('%s: positional argument %d is a %s, not a tensor (compile-time constants are '
                                'passed by keyword)' % (self.name, position, type(arg).__name__))
            resolved.append(arg)
        return resolved, types

    def _trace_gradient(self, input_types, output_types, constants):
        """Operator graph of the registered gradient function for these types, or None when the function declines
        (returns None for some input).  Its leaves are placeholders in signature order: the operator's inputs,
        then one gradient per operator output.  Every returned gradient must have its input's tensor type
        (TypeError otherwise, opveclib/operator.py:512-523)."""
        leaves = [GradientPlaceholder(t.shape, t.dtype) for t in list(input_types) + list(output_types)]
        returned = self.grad_function(*leaves, **constants)
        if returned is None or isinstance(returned, (Operator, OperatorOutput)):
            returned = [returned]
        returned = list(returned)
        if any(g is None for g in returned):
            return None
        for index, (g, expected) in enumerate(zip(returned, input_types)):
            if isinstance(g, Operator) and len(g.output_types) != 1:
                raise TypeError('gradient %d of %s is an operator with %d outputs: index the one that is meant'
                                % (index, self.name, len(g.output_types)))
            got = TensorType.like(_resolve_output(g))
            if got != expected:
                raise TypeError('gradient %d of %s has type %s, its input has type %s'
                                % (index, self.name, got, expected))
        return build_op_dag(*returned, leaf_order=leaves)

    def __call__(self, *inputs, **defined_constants):
        """Trace the operator for these arguments: positional arguments are tensors (arrays, operator outputs,
        placeholders), keyword arguments override the constants' defaults."""
        tensor_names, constants, variadic = self._parameters()
        constants.update(defined_constants)
        if self.forbid_none_valued_constants:
            unset = sorted(k for k, v in constants.items() if v is None)
            if unset:
                raise ValueError('%s: constant(s) %s are None, i.e. not set (decorate the operator with '
                                 'forbid_none_valued_constants=False if None is a meaningful value)'
                                 % (self.name, ', '.join(unset)))
        resolved, input_types = self._tensor_arguments(inputs)
        if len(input_types) != len(tensor_names) and not variadic:
            hint = ''
            if len(input_types) < len(tensor_names):
                hint = '; missing: ' + ', '.join(tensor_names[len(input_types):])
            raise TypeError('%s takes %d tensor argument(s) (%s) but got %d%s'
                            % (self.name, len(tensor_names), ', '.join(tensor_names), len(input_types), hint))
        kernel = trace_function(self.op_function, input_types, constants, self.name)
        # operators applied while a gradient is being traced do not get gradients of their own
        from_gradient = any(isinstance(a, GradientPlaceholder) or getattr(a, 'from_gradient', False) for a in inputs)
        grad_dag = None
        if self.grad_function is not None and not from_gradient:
            grad_dag = self._trace_gradient(input_types, kernel.output_types, constants)
        return Operator(kernel, resolved, grad_dag, from_gradient, self.name, self, dict(defined_constants))

    def add_grad(self, grad_function):
        if self.grad_function is not None:
            raise ValueError('Gradient function is already defined for operator ' + str(self.name) + '.')
        self.grad_function = grad_function


def _check_reassignment(op_function):
    """Reject python ``=`` re-binding of a name that was bound to ``variable(...)``: such a statement would
    silently drop the assignment from the generated code; ``<<=`` is the assignment operator of the language
    (opveclib/operator.py:566-641)."""
    variable_names = set()
    by_line = {}
    instructions = list(dis.get_instructions(op_function))
    line = None
    for ins in instructions:
        starts = getattr(ins, 'line_number', None)
        if starts is None:
            starts = ins.starts_line if isinstance(ins.starts_line, int) and not isinstance(
                ins.starts_line, bool) else None
        if starts is not None:
            line = starts
        by_line.setdefault(line, []).append(ins)
    for line in sorted(k for k in by_line if k is not None):
        group = by_line[line]
        for pos, ins in enumerate(group):
            if ins.opname != 'STORE_FAST':
                continue
            before = group[:pos]
            is_variable = any(p.opname in ('LOAD_GLOBAL', 'LOAD_ATTR', 'LOAD_METHOD', 'LOAD_NAME', 'LOAD_DEREF')
                              and p.argval == 'variable' for p in before)
            prev = before[-1] if before else None
            has_lshift = prev is not None and (prev.opname == 'INPLACE_LSHIFT' or
                                               (prev.opname == 'BINARY_OP' and '<<=' in str(prev.argrepr)))
            name = ins.argval
            if name in variable_names and not has_lshift:
                raise SyntaxError('Cannot reassign to symbol "' + str(name) + '" in operator "' +
                                  op_function.__name__ + '" because it refers to an OVL variable. Use the '
                                  '<<= operator to assign to OVL variables. \n  File "' +
                                  op_function.__code__.co_filename + '", line ' + str(line))
            if is_variable:
                variable_names.add(name)


def operator(forbid_none_valued_constants=True, name=None):
    """Decorator that turns a DSL function into an operator generator.  Positional parameters are tensor
    inputs; parameters with defaults are compile-time constants passed by keyword."""
    def wrapper(op_function):
        _check_reassignment(op_function)
        return OpGenerator(op_function, forbid_none_valued_constants, name)
    return wrapper


def gradient(op_function):
    """Decorator that registers the gradient of ``op_function``: a function of (inputs..., output grads...,
    **constants) returning one gradient per input, itself an operator or a python function composing
    operators."""
    if not isinstance(op_function, OpGenerator):
        raise TypeError('gradient decorator argument must be a function decorated as an operator')

    def wrapper(grad_function):
        if isinstance(grad_function, OpGenerator):
            def resolved(*args, **defaults):
                op = grad_function(*args, **defaults)
                return [op[i] for i in range(len(op.output_types))]
        else:
            resolved = grad_function
        op_function.add_grad(resolved)
        try:
            resolved.__name__ = grad_function.__name__
            resolved.__doc__ = grad_function.__doc__
        except AttributeError:
            pass
        return resolved
    return wrapper


class InputRef(object):
    """Where one operator input comes from: a leaf (``dag_input_index``) or another operator's output."""
    __slots__ = ('is_leaf', 'dag_input_index', 'op_index', 'op_output_index')

    def __init__(self, is_leaf, dag_input_index=None, op_index=None, op_output_index=None):
        self.is_leaf = is_leaf
        self.dag_input_index = dag_input_index
        self.op_index = op_index
        self.op_output_index = op_output_index

    def key(self):
        return ('L', self.dag_input_index) if self.is_leaf else ('O', self.op_index, self.op_output_index)


class OpDAG(object):
    """Operators in dependency order with their input references; mirrors the reference's ``OperatorDAG``
    message (opveclib/language.proto:406-429).

    kernels      KernelIR per operator
    references   list (per operator) of InputRef
    inputs       leaf input objects (arrays / placeholders), ``input_types`` their TensorTypes
    outputs      list of (op_index, op_output_index)
    grad_dags    per operator gradient OpDAG or None
    """

    def __init__(self, kernels, references, inputs, input_types, outputs, grad_dags):
        self.kernels = kernels
        self.references = references
        self.inputs = inputs
        self.input_types = input_types
        self.outputs = outputs
        self.grad_dags = grad_dags

    def text(self):
        parts = []
        for k, refs in zip(self.kernels, self.references):
            parts.append(k.text() + '|' + ';'.join(str(r.key()) for r in refs))
        parts.append('in:' + ';'.join(str(t) for t in self.input_types))
        parts.append('out:' + ';'.join(str(o) for o in self.outputs))
        return '\n'.join(parts)


def build_op_dag(*outputs, **kwargs):
    """Collect every operator the requested outputs depend on (depth first), order them by depth so producers
    precede consumers, and record leaf inputs in discovery order (opveclib/operator.py:679-806).

    ``leaf_order`` (keyword): a list of leaf objects that fixes the graph's input signature; leaves found are
    mapped onto it by identity and leaves never used stay in the signature."""
    leaf_order = kwargs.pop('leaf_order', None)
    ops, op_ids, depth, input_indices = [], {}, [], []
    dag_inputs, dag_input_ids = [], {}
    if leaf_order is not None:
        for leaf in leaf_order:
            dag_input_ids[id(leaf)] = len(dag_inputs)
            dag_inputs.append(leaf)

    def traverse(node):
        if not isinstance(node, Operator):
            raise TypeError()
        if id(node) in op_ids:
            return op_ids[id(node)]
        index = len(ops)
        op_ids[id(node)] = index
        ops.append(node)
        depth.append(None)
        input_indices.append(None)
        cur, max_depth = [], -1
        for cur_input in node.inputs:
            if isinstance(cur_input, (Operator, OperatorOutput)):
                resolved = _resolve_output(cur_input)
                parent_index = traverse(resolved.parent)
                max_depth = max(max_depth, depth[parent_index])
                cur.append((parent_index, resolved.index, None))
            else:
                if id(cur_input) not in dag_input_ids:
                    if leaf_order is not None:
                        raise ValueError('Gradient function used a tensor that is not one of its arguments.')
                    dag_input_ids[id(cur_input)] = len(dag_inputs)
                    dag_inputs.append(cur_input)
                cur.append((None, None, dag_input_ids[id(cur_input)]))
        input_indices[index] = cur
        depth[index] = max_depth + 1
        return index

    output_indices = []
    for dag_output in outputs:
        cur_output = _resolve_output(dag_output)
        output_indices.append((traverse(cur_output.parent), cur_output.index))

    new_to_old = np.argsort(depth, kind='stable')
    old_to_new = np.argsort(new_to_old, kind='stable')
    kernels, references, grad_dags = [], [], []
    for old_index in new_to_old:
        op = ops[old_index]
        kernels.append(op.kernel)
        grad_dags.append(op.grad_dag)
        refs = []
        for parent_index, output_index, dag_input_index in input_indices[old_index]:
            if parent_index is None:
                refs.append(InputRef(True, dag_input_index=dag_input_index))
            else:
                refs.append(InputRef(False, op_index=int(old_to_new[parent_index]),
                                     op_output_index=int(output_index)))
        references.append(refs)
    dag_outputs = [(int(old_to_new[p]), int(o)) for p, o in output_indices]
    input_types = [TensorType.like(x) for x in dag_inputs]
    return OpDAG(kernels, references, dag_inputs, input_types, dag_outputs, grad_dags)
