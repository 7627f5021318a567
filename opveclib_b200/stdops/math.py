"""Component-wise math, split/concat and broadcasting binary operators with their gradients.

Operator set, argument conventions and per-element arithmetic follow opveclib/stdops/math.py:15-392: unary
operators map ``f`` over the tensor; binary operators take two tensors of equal shape or one tensor and a size-1
tensor that is broadcast; ``split``/``concat`` cut and join along one axis.  The infix operators of operator
outputs (``a + b``, ``-a``, ``a < b`` ...) are registered here.
"""
from .. import expr as E
from ..dtypes import uint8, uint16, uint32, uint64
from ..opgraph import operator, gradient, OperatorOutput


def _map1(arg, func):
    out = E.output(arg.shape, arg.dtype)
    pos = E.position_in(arg.shape)
    out[pos] = func(arg[pos])
    return out


def _map1_grad(arg, grad_above, func):
    out = E.output(arg.shape, arg.dtype)
    pos = E.position_in(arg.shape)
    out[pos] = func(arg[pos], grad_above[pos])
    return out


@operator()
def neg(arg):
    if arg.dtype in (uint8, uint16, uint32, uint64):
        raise TypeError('Cannot negate an unsigned tensor.')
    return _map1(arg, lambda x: -x)


@gradient(neg)
@operator()
def neg_grad(arg, grad_above):
    return _map1_grad(arg, grad_above, lambda x, dz: -dz)


OperatorOutput.register_magic_method('neg', neg)


@operator()
def tanh(arg):
    return _map1(arg, lambda x: E.tanh(x))


@gradient(tanh)
@operator()
def tanh_grad(arg, grad_above):
    return _map1_grad(arg, grad_above, lambda x, dz: (1 - E.tanh(x) * E.tanh(x)) * dz)


@operator()
def sin(arg):
    return _map1(arg, lambda x: E.sin(x))


@gradient(sin)
@operator()
def sin_grad(arg, grad_above):
    return _map1_grad(arg, grad_above, lambda x, dz: E.cos(x) * dz)


@operator()
def cos(arg):
    return _map1(arg, lambda x: E.cos(x))


@gradient(cos)
@operator()
def cos_grad(arg, grad_above):
    return _map1_grad(arg, grad_above, lambda x, dz: -E.sin(x) * dz)


@operator()
def tan(arg):
    return _map1(arg, lambda x: E.tan(x))


@gradient(tan)
@operator()
def tan_grad(arg, grad_above):
    return _map1_grad(arg, grad_above, lambda x, dz: (1 / (E.cos(x) * E.cos(x))) * dz)


@operator()
def sigmoid(arg):
    return _map1(arg, lambda x: 1 / (1 + E.exp(-x)))


@gradient(sigmoid)
@operator()
def sigmoid_grad(arg, grad_above):
    grad = E.output_like(arg)
    pos = E.position_in(arg.shape)
    # outside (-50, 50) exp(-x) over/underflows; the derivative is taken as zero there
    inside = E.logical_and(arg[pos] > -50, arg[pos] < 50)
    result = E.variable(0, arg.dtype)
    with E.if_(inside):
        e = E.exp(-arg[pos])
        result <<= e / ((1 + e) * (1 + e))
    grad[pos] = result * grad_above[pos]
    return grad


@operator()
def split(arg, split_dim=None, num_split=None):
    """Cut ``arg`` into ``num_split`` equal parts along ``split_dim``; one output per part."""
    part, remainder = divmod(arg.shape[split_dim], num_split)
    if remainder != 0:
        raise ValueError('num_split must evenly divide the axis')
    out_shape = [part if d == split_dim else n for d, n in enumerate(arg.shape)]
    pos = E.position_in(out_shape)
    outputs = []
    for n in range(num_split):
        outputs.append(E.output(out_shape, arg.dtype))
        src = [n * part + pos[d] if d == split_dim else pos[d] for d in range(arg.rank)]
        outputs[n][pos] = arg[src]
    return outputs


@operator()
def concat(*args, **constants):
    """Join tensors along ``concat_dim``.  Equal-shaped parts use one worker per part element; parts of
    different extent use one worker per output element and select the part by range tests."""
    concat_dim = constants['concat_dim']
    ref = args[0]
    bounds = [0]
    all_same = True
    for arg in args:
        assert arg.rank == ref.rank
        assert arg.dtype == ref.dtype
        if arg.shape != ref.shape:
            all_same = False
        bounds.append(bounds[-1] + arg.shape[concat_dim])
        for d in range(ref.rank):
            if d != concat_dim:
                assert arg.shape[d] == ref.shape[d]

    if all_same:
        out_shape = [len(args) * n if d == concat_dim else n for d, n in enumerate(ref.shape)]
        pos = E.position_in(ref.shape)
        out = E.output(out_shape, ref.dtype)
        for k, arg in enumerate(args):
            dst = [k * ref.shape[d] + pos[d] if d == concat_dim else pos[d] for d in range(ref.rank)]
            out[dst] = arg[pos]
    else:
        out_shape = [bounds[-1] if d == concat_dim else n for d, n in enumerate(ref.shape)]
        out = E.output(out_shape, ref.dtype)
        pos = E.position_in(out_shape)
        for k, arg in enumerate(args):
            lo, hi = bounds[k], bounds[k + 1]
            along = pos[concat_dim]
            with E.if_(E.logical_and(along >= lo, along < hi)):
                src = [along - lo if d == concat_dim else pos[d] for d in range(ref.rank)]
                out[pos] = arg[src]
    return out


@gradient(split)
def split_grad(arg, *grads_above, **constants):
    return concat(*grads_above, concat_dim=constants['split_dim'])


@gradient(concat)
def concat_grad(*args, **constants):
    inputs, grad_above = args[:-1], args[-1]
    first = inputs[0].tensor_type
    if all(i.tensor_type == first for i in inputs[1:]):
        parts = split(grad_above, split_dim=constants['concat_dim'], num_split=len(inputs))
        return [parts[n] for n in range(len(inputs))]
    return [None] * len(inputs)


def _positions(lhs, rhs):
    """(lhs index, rhs index, full index) for equal shapes or a size-1 operand on either side."""
    if lhs.size == 1 and rhs.size > 1:
        full = E.position_in(rhs.shape)
        return [0] * lhs.rank, full, full, rhs
    if lhs.size > 1 and rhs.size == 1:
        full = E.position_in(lhs.shape)
        return full, [0] * rhs.rank, full, lhs
    if lhs.shape == rhs.shape:
        full = E.position_in(lhs.shape)
        return full, full, full, lhs
    raise TypeError('Binary operands must either be the same shape, or at least one must be a scalar.')


def _map2(lhs, rhs, fcn):
    if lhs.dtype != rhs.dtype:
        raise TypeError('Binary operator input dtypes must be the same.')
    # the output is declared before the position, as operands of the larger shape define both
    if lhs.size == 1 and rhs.size > 1:
        out = E.output_like(rhs)
    elif lhs.size > 1 and rhs.size == 1:
        out = E.output_like(lhs)
    elif lhs.shape == rhs.shape:
        out = E.output_like(lhs)
    else:
        raise TypeError('Binary operands must either be the same shape, or at least one must be a scalar.')
    lhs_pos, rhs_pos, out_pos, _ = _positions(lhs, rhs)
    out[out_pos] = fcn(lhs[lhs_pos], rhs[rhs_pos])
    return out


def _map2_grad(lhs, rhs, grad, fcn):
    if lhs.dtype != rhs.dtype or lhs.dtype != grad.dtype:
        raise TypeError('Binary operator input and gradient dtypes must be the same.')
    lhs_grad = E.output_like(lhs)
    rhs_grad = E.output_like(rhs)
    lhs_pos, rhs_pos, grad_pos, _ = _positions(lhs, rhs)
    lhs_val, rhs_val = fcn(lhs[lhs_pos], rhs[rhs_pos], grad[grad_pos])
    lhs_grad[lhs_pos] = lhs_val
    rhs_grad[rhs_pos] = rhs_val
    return lhs_grad, rhs_grad


@operator()
def add(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x + y)


@gradient(add)
@operator()
def add_grad(lhs, rhs, grad_above):
    return _map2_grad(lhs, rhs, grad_above, lambda x, y, dz: (dz, dz))


@operator()
def sub(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x - y)


@gradient(sub)
@operator()
def sub_grad(lhs, rhs, grad_above):
    return _map2_grad(lhs, rhs, grad_above, lambda x, y, dz: (dz, -dz))


@operator()
def mul(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x * y)


@gradient(mul)
@operator()
def mul_grad(lhs, rhs, grad_above):
    return _map2_grad(lhs, rhs, grad_above, lambda x, y, dz: (y * dz, x * dz))


@operator()
def div(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x / y)


@gradient(div)
@operator()
def div_grad(lhs, rhs, grad_above):
    return _map2_grad(lhs, rhs, grad_above, lambda x, y, dz: (dz / y, -x / (y * y) * dz))


@operator()
def mod(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x % y)


@operator()
def equal(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x == y)


@operator()
def not_equal(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x != y)


@operator()
def less(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x < y)


@operator()
def less_equal(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x <= y)


@operator()
def greater(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x > y)


@operator()
def greater_equal(lhs, rhs):
    return _map2(lhs, rhs, lambda x, y: x >= y)


for _key, _op in (('add', add), ('sub', sub), ('mul', mul), ('div', div), ('mod', mod), ('eq', equal),
                  ('ne', not_equal), ('lt', less), ('le', less_equal), ('gt', greater), ('ge', greater_equal)):
    OperatorOutput.register_magic_method(_key, _op)
