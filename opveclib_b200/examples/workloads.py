"""Benchmark and smoke workloads written against the operator API.

The operators and chains of the benchmark configurations: the README's cyclic shift, the four-operator chain
``expm1(log1p(|x|)) * 0.5 + x``, the sixteen-operator chain, element-wise building blocks, per-worker reduction
loops (dot product, matrix-vector product, row products, column sums) and operators that read or write a
transposed operand.  Every function takes the implementation as a namespace ``ns`` (``ns.ovl`` is the operator
API, ``ns.expm1`` / ``ns.log1p`` / ``ns.cumsum`` ... the example operators), so the same definitions can be
instantiated with this package (:func:`namespace`) and, when golden vectors are recorded, with the reference
package - the operator API is the same, which is the point of a drop-in backend.
"""
import types


def namespace():
    """This package behind the namespace the workloads use."""
    import opveclib_b200 as ovl
    from opveclib_b200 import examples, stdops
    return types.SimpleNamespace(ovl=ovl, stdops=stdops, cumsum=examples.cumsum, cumprod=examples.cumprod,
                                 accumulate=examples.accumulate, expm1=examples.expm1, log1p=examples.log1p,
                                 lstm=examples.lstm, lstm_grad=examples.lstm_grad, conv_1d=examples.conv_1d)


# ---------------------------------------------------------------------------------------------------------
# user-level operators of the benchmark configurations, built per implementation
_cache = {}


def user_ops(ns):
    key = id(ns.ovl)
    if key in _cache:
        return _cache[key]
    ovl = ns.ovl

    @ovl.operator()
    def shift_cyclic(input_tensor):
        assert input_tensor.rank == 1
        output_tensor = ovl.output_like(input_tensor)
        wg_position = ovl.position_in(input_tensor.shape)
        input_element = input_tensor[wg_position]
        output_position = (wg_position[0] + 1) % input_tensor.size
        output_tensor[output_position] = input_element
        return output_tensor

    @ovl.operator()
    def absolute(x):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = ovl.absolute(x[pos])
        return out

    @ovl.operator()
    def halfplus(t, x):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = t[pos] * 0.5 + x[pos]
        return out

    @ovl.operator()
    def ew_exp(x):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = ovl.exp(x[pos])
        return out

    @ovl.operator()
    def ew_tanh(x):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = ovl.tanh(x[pos])
        return out

    @ovl.operator()
    def ew_add(x, y):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = x[pos] + y[pos]
        return out

    @ovl.operator()
    def ew_mul(x, y):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = x[pos] * y[pos]
        return out

    @ovl.operator()
    def ew_addc(x, c=None):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = x[pos] + c
        return out

    @ovl.operator()
    def ew_mulc(x, c=None):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = x[pos] * c
        return out

    @ovl.operator()
    def where_greater(a, b):
        # a where a > b, else b
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        r = ovl.variable(0, a.dtype)
        with ovl.if_(a[pos] > b[pos]):
            r <<= a[pos]
        with ovl.else_():
            r <<= b[pos]
        out[pos] = r
        return out

    @ovl.operator()
    def dot(input0, input1):
        # per-row dot product with a float64 accumulator (opveclib/test/test_dot_product.py:18-34)
        num_vectors = input0.shape[0]
        dot_out = ovl.output(num_vectors, input0.dtype)
        pos = ovl.position_in(num_vectors)[0]
        accum = ovl.variable(0.0, ovl.float64)
        num_elements = ovl.variable(input0.shape[1], ovl.uint32)
        for i in ovl.arange(num_elements):
            accum <<= accum + input0[pos, i] * input1[pos, i]
        dot_out[pos] = accum
        return dot_out

    @ovl.operator()
    def matvec(mat, vec):
        # matrix-vector product, one worker per row (documentation/programming.rst:320-344)
        assert mat.rank == 2 and vec.rank == 1 and mat.shape[1] == vec.shape[0] and mat.dtype == vec.dtype
        rows, cols = mat.shape[0], mat.shape[1]
        y = ovl.output(rows, mat.dtype)
        row = ovl.position_in(rows)[0]
        accum = ovl.variable(0, mat.dtype)
        for col in ovl.arange(cols):
            accum <<= accum + mat[row, col] * vec[col]
        y[row] = accum
        return y

    @ovl.operator()
    def rowprod_scaled(x, scale):
        # product over the last axis of a rank-3 tensor, then scaled: statements after the loop use the result
        out = ovl.output([x.shape[0], x.shape[1]], x.dtype)
        pos = ovl.position_in([x.shape[0], x.shape[1]])
        accum = ovl.variable(1, x.dtype)
        for i in ovl.arange(x.shape[2]):
            accum <<= x[pos[0], pos[1], i] * accum
        out[pos] = accum * scale[pos[1]]
        return out

    @ovl.operator()
    def transpose(a):
        # the operand is read along the workgroup's first axis: neighbouring workers are a row apart in memory
        out = ovl.output([a.shape[1], a.shape[0]], a.dtype)
        pos = ovl.position_in(out.shape)
        out[pos] = a[pos[1], pos[0]]
        return out

    @ovl.operator()
    def transpose_axpy(a, b, alpha=None):
        # b and the output share the layout; a comes in transposed
        out = ovl.output_like(b)
        pos = ovl.position_in(b.shape)
        out[pos] = a[pos[1], pos[0]] * alpha + b[pos]
        return out

    @ovl.operator()
    def colsum(a):
        # one worker per column folds the rows: strided along the loop, contiguous across workers
        out = ovl.output([a.shape[1]], a.dtype)
        col = ovl.position_in([a.shape[1]])[0]
        accum = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[0]):
            accum <<= accum + a[i, col]
        out[col] = accum
        return out

    @ovl.operator()
    def rowsum(a):
        # one worker per row folds the row in order: short rows are staged in shared memory, long ones reduced by a warp
        out = ovl.output([a.shape[0]], a.dtype)
        row = ovl.position_in([a.shape[0]])[0]
        accum = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[1]):
            accum <<= accum + a[row, i]
        out[row] = accum
        return out

    @ovl.operator()
    def row_normalise(a):
        # every row divided by its sum: one loop that reads the row, a second one that reads and writes it
        out = ovl.output_like(a)
        row = ovl.position_in([a.shape[0]])[0]
        accum = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[1]):
            accum <<= accum + a[row, i]
        for i in ovl.arange(a.shape[1]):
            out[row, i] = a[row, i] / accum
        return out

    ops = types.SimpleNamespace(transpose=transpose, transpose_axpy=transpose_axpy, colsum=colsum, rowsum=rowsum,
                                row_normalise=row_normalise,
                                shift_cyclic=shift_cyclic, absolute=absolute, halfplus=halfplus, ew_exp=ew_exp,
                                dot=dot, matvec=matvec, rowprod_scaled=rowprod_scaled,
                                ew_tanh=ew_tanh, ew_add=ew_add, ew_mul=ew_mul, ew_addc=ew_addc, ew_mulc=ew_mulc,
                                where_greater=where_greater)
    _cache[key] = ops
    return ops


def c1_chain(ns, x):
    """y = expm1(log1p(|x|)) * 0.5 + x as four operators."""
    u = user_ops(ns)
    return u.halfplus(ns.expm1(ns.log1p(u.absolute(x))), x)


def chain16(ns, x):
    """Sixteen element-wise operators (add, mul, exp, log1p, expm1, tanh, where on a comparison) over one
    tensor; values stay finite for inputs in [-2, 2]."""
    u = user_ops(ns)
    a = u.ew_mulc(x, c=0.5)
    b = u.ew_tanh(a)
    c = u.ew_exp(b)
    d = ns.log1p(c)
    e = u.ew_add(d, x)
    f = ns.expm1(a)
    g = u.ew_mul(f, b)
    h = u.where_greater(g, e)
    i = u.ew_addc(h, c=1.0)
    j = u.ew_mul(i, i)
    k = ns.log1p(j)
    l = u.ew_tanh(k)
    m = u.ew_exp(l)
    n = u.ew_mulc(m, c=0.25)
    o = ns.expm1(n)
    return u.ew_add(o, e)


def chain16_light(ns, x):
    """Sixteen element-wise operators without transcendentals (add, mul, where on a comparison): the same graph
    shape as chain16 with a body light enough to be limited by memory bandwidth."""
    u = user_ops(ns)
    a = u.ew_mulc(x, c=0.5)
    b = u.ew_addc(a, c=1.0)
    c = u.ew_mul(b, a)
    d = u.ew_add(c, x)
    e = u.where_greater(d, a)
    f = u.ew_mulc(e, c=0.25)
    g = u.ew_mul(f, b)
    h = u.ew_add(g, d)
    i = u.ew_addc(h, c=-0.5)
    j = u.ew_mul(i, i)
    k = u.where_greater(j, h)
    l = u.ew_mulc(k, c=0.125)
    m = u.ew_add(l, e)
    n = u.ew_mul(m, a)
    o = u.ew_addc(n, c=2.0)
    return u.ew_add(o, x)


def stdops_lstm(ns, gates, c):
    """The LSTM cell composed from the operator library: split the gates, sigmoid / tanh, multiply, add
    (the graph of opveclib/test/test_operator_merge.py:311-321; gate order i, j, f, o as in lstm/lstm.py:45-48,
    forget bias 0).  Returns [new_c, new_h]."""
    so = ns.stdops
    i, j, f, o = so.split(gates, split_dim=1, num_split=4)
    new_c = so.mul(c, so.sigmoid(f)) + so.sigmoid(i) * so.tanh(j)
    new_h = so.tanh(new_c) * so.sigmoid(o)
    return [new_c, new_h]
