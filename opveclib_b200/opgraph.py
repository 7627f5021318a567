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


class OperatorOutput(object):
    """An un-evaluated output tensor of an :class:`Operator`.  Infix arithmetic and comparisons between
    outputs dispatch to the standard operator library registered with :meth:`register_magic_method`."""
    __array_priority__ = 1
    _builtin_ops = {}

    @staticmethod
    def register_magic_method(key, value):
        OperatorOutput._builtin_ops[key] = value

    def __init__(self, parent, index):
        if not isinstance(parent, Operator):
            raise TypeError('parent must be an Operator')
        if not isinstance(index, int):
            raise TypeError('index must be an int')
        self.parent = parent
        self.index = index
        self.tensor_type = parent.output_types[index]
        self.shape = self.tensor_type.shape
        self.dtype = self.tensor_type.dtype
        self.size = self.tensor_type.size
        self.rank = self.tensor_type.rank

    @property
    def from_gradient(self):
        return self.parent.from_gradient

    def _call(self, key, *args):
        return OperatorOutput._builtin_ops[key](*args)

    def __add__(self, other):
        return self._call('add', self, other)

    def __radd__(self, other):
        return self._call('add', other, self)

    def __sub__(self, other):
        return self._call('sub', self, other)

    def __rsub__(self, other):
        return self._call('sub', other, self)

    def __mul__(self, other):
        return self._call('mul', self, other)

    def __rmul__(self, other):
        return self._call('mul', other, self)

    def __truediv__(self, other):
        return self._call('div', self, other)

    def __rtruediv__(self, other):
        return self._call('div', other, self)

    __div__ = __truediv__
    __rdiv__ = __rtruediv__

    def __mod__(self, other):
        return self._call('mod', self, other)

    def __rmod__(self, other):
        return self._call('mod', other, self)

    def __eq__(self, other):
        return self._call('eq', self, other)

    def __ne__(self, other):
        return self._call('ne', self, other)

    def __lt__(self, other):
        return self._call('lt', self, other)

    def __le__(self, other):
        return self._call('le', self, other)

    def __gt__(self, other):
        return self._call('gt', self, other)

    def __ge__(self, other):
        return self._call('ge', self, other)

    def __neg__(self):
        return self._call('neg', self)

    def __bool__(self):
        raise SyntaxError('Cannot resolve operator values at interpretation time.')

    __hash__ = object.__hash__


class GradientPlaceholder(object):
    """Stands for an operator input or an output gradient while a gradient function is traced."""

    def __init__(self, shape, dtype):
        self.tensor_type = TensorType(shape, dtype)
        self.rank = self.tensor_type.rank
        self.shape = list(shape)
        self.dtype = self.tensor_type.dtype
        self.size = self.tensor_type.size


class Operator(object):
    """A lazily evaluated operator application: a traced kernel plus where its inputs come from."""
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
        for i in range(len(self.output_types)):
            yield OperatorOutput(self, i)

    def check_binary(self):
        if len(self.output_types) != 1:
            raise SyntaxError('Cannot use binary infix operators on multi-output operators. '
                              'Explicitly index an output.')

    @property
    def shape(self):
        self.check_binary()
        return self.output_types[0].shape

    @property
    def dtype(self):
        self.check_binary()
        return self.output_types[0].dtype

    def __add__(self, other):
        self.check_binary()
        return self[0] + other

    def __radd__(self, other):
        self.check_binary()
        return other + self[0]

    def __sub__(self, other):
        self.check_binary()
        return self[0] - other

    def __rsub__(self, other):
        self.check_binary()
        return other - self[0]

    def __mul__(self, other):
        self.check_binary()
        return self[0] * other

    def __rmul__(self, other):
        self.check_binary()
        return other * self[0]

    def __truediv__(self, other):
        self.check_binary()
        return self[0] / other

    def __rtruediv__(self, other):
        self.check_binary()
        return other / self[0]

    __div__ = __truediv__
    __rdiv__ = __rtruediv__

    def __mod__(self, other):
        self.check_binary()
        return self[0] % other

    def __rmod__(self, other):
        self.check_binary()
        return other % self[0]

    def __eq__(self, other):
        self.check_binary()
        return self[0] == other

    def __ne__(self, other):
        self.check_binary()
        return self[0] != other

    def __lt__(self, other):
        self.check_binary()
        return self[0] < other

    def __le__(self, other):
        self.check_binary()
        return self[0] <= other

    def __gt__(self, other):
        self.check_binary()
        return self[0] > other

    def __ge__(self, other):
        self.check_binary()
        return self[0] >= other

    def __neg__(self):
        self.check_binary()
        return -self[0]

    __hash__ = object.__hash__


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

    def __call__(self, *inputs, **defined_constants):
        from_gradient = False
        for inp in inputs:
            if getattr(inp, 'from_gradient', False) or isinstance(inp, GradientPlaceholder):
                from_gradient = True

        spec = inspect.getfullargspec(self.op_function)
        func_args, func_varargs, func_defaults = spec.args, spec.varargs, spec.defaults
        if func_defaults is None:
            input_names = func_args
            constants = dict(defined_constants)
        else:
            input_names = func_args[:-len(func_defaults)]
            constants = dict(zip(func_args[-len(func_defaults):], func_defaults))
            constants.update(defined_constants)

        if self.forbid_none_valued_constants:
            for key in constants:
                if constants[key] is None:
                    raise ValueError(self.name + ' argument ' + key + ' is None, which implies an unset '
                                     'constant.\n  If a None constant is meaningful for this operator, the '
                                     'operator should be defined with the appropriate decorator flag.')

        resolved_inputs = []
        input_types = []
        for inp_n, inp in enumerate(inputs):
            try:
                inp = _resolve_output(inp)
            except TypeError:
                pass
            try:
                input_types.append(TensorType.like(inp))
            except (AttributeError, TypeError):
                raise TypeError('Unexpectedly received a ' + inp.__class__.__name__ +
                                ' instead of a tensor at argument position ' + str(inp_n + 1) +
                                ' in the call to ' + self.name + '.  Should this argument be passed as a '
                                'constant (keyword argument) instead?')
            resolved_inputs.append(inp)

        num_inputs = len(input_types)
        if len(input_names) != num_inputs and func_varargs is None:
            err_msg = '\n' + self.name + ' function signature expects ' + str(len(input_names)) + \
                ' input tensor argument(s):\n' + str(input_names) + '\n'
            err_msg += 'but was supplied with ' + str(num_inputs) + '.\n'
            if len(input_names) > num_inputs:
                remaining_names = input_names[num_inputs - len(input_names):]
                err_msg += 'Should ' + str(remaining_names) + ' be passed to constructor as constant?'
            raise TypeError(err_msg)

        kernel = trace_function(self.op_function, input_types, constants, self.name)
        output_types = kernel.output_types

        grad_dag = None
        if self.grad_function is not None and not from_gradient:
            grad_inputs = [GradientPlaceholder(t.shape, t.dtype) for t in input_types]
            grad_inputs += [GradientPlaceholder(t.shape, t.dtype) for t in output_types]
            grad_outputs = self.grad_function(*grad_inputs, **constants)
            if isinstance(grad_outputs, (Operator, OperatorOutput)) or grad_outputs is None:
                grad_outputs = [grad_outputs]
            grad_outputs = list(grad_outputs)
            if not any(g is None for g in grad_outputs):
                for gi, g in enumerate(grad_outputs):
                    if isinstance(g, Operator) and len(g.output_types) != 1:
                        raise TypeError('A multi-output operator was returned from a gradient function, '
                                        'but the meaning of this is ambiguous: explicitly index each '
                                        'output from operator: ' + str(g.name))
                    cur_input_type = input_types[gi]
                    cur_grad_type = TensorType.like(_resolve_output(g))
                    if cur_input_type != cur_grad_type:
                        raise TypeError('Gradient output index ' + str(gi) + ', with TensorType: ' +
                                        str(cur_grad_type) + ' is inconsistent with operator input index ' +
                                        str(gi) + ', with TensorType: ' + str(cur_input_type))
                # the gradient graph's leaf inputs are the placeholders, in signature order: operator inputs
                # first, then one gradient per operator output
                grad_dag = build_op_dag(*grad_outputs, leaf_order=grad_inputs)

        return Operator(kernel, resolved_inputs, grad_dag, from_gradient, self.name, self, dict(defined_constants))

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
