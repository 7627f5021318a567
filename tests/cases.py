"""Workload definitions shared by the parity tests and by the script that records golden vectors.

Every case is written once against the operator API and instantiated twice: with this package (``impl()``) in
the tests, and with the reference package inside ``tests/golden/make_golden.py`` - the operator API is the same,
which is the point of a drop-in backend.  A case returns ``(outputs, inputs)``: the operator outputs to
evaluate and the numpy leaf arrays (for the fixture file).  Inputs are seeded; sizes are small enough for the
CPU oracle and the fixtures, with shapes chosen to hit vector tails, tile boundaries and broadcast paths.
"""
import types

import numpy as np

from opveclib_b200.examples.workloads import (namespace as impl, user_ops, c1_chain, chain16,  # noqa: F401
                                               chain16_light, stdops_lstm)


# ---------------------------------------------------------------------------------------------------------
def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def case_shift_readme(ns):
    x = _f32([0, 1, 2, 3, 4])
    return [user_ops(ns).shift_cyclic(x)], [x]


def case_shift_1031(ns):
    x = _f32(np.random.RandomState(11).uniform(-1, 1, 1031))
    return [user_ops(ns).shift_cyclic(x)], [x]


def case_shift_4096(ns):
    x = _f32(np.random.RandomState(12).uniform(-1, 1, 4096))
    return [user_ops(ns).shift_cyclic(x)], [x]


def case_c1_chain(ns):
    x = np.random.RandomState(1).uniform(-1, 1, 4100)
    x[:6] = [0.0, 1e-10, -1e-10, 1.0, -1.0, 0.5]
    x = _f32(x)
    return [c1_chain(ns, x)], [x]


def case_c1_chain_odd(ns):
    x = _f32(np.random.RandomState(2).uniform(-1, 1, 1023))
    return [c1_chain(ns, x)], [x]


def case_expm1_f64(ns):
    x = np.array([1e-10, -1e-10, 0.0, np.inf, 1.0, -50.0, 1e-99, 700.0])
    return [ns.expm1(x)], [x]


def case_log1p_f64(ns):
    x = np.array([1e-99, -1e-99, 0.0, np.inf, 1.0, -0.5, 1e-10, 1e10])
    return [ns.log1p(x)], [x]


def case_cumsum_doctest(ns):
    a = np.arange(1, 6)
    b = np.arange(1, 16).reshape(3, 5)
    return [ns.cumsum(a), ns.cumsum(b, axis=0), ns.cumprod(a), ns.cumprod(b, axis=0)], [a, b]


def case_accumulate_555(ns):
    x = np.random.RandomState(3).uniform(0.5, 1.5, (5, 5, 5))
    outs = []
    for axis in range(3):
        outs += [ns.cumsum(x, axis=axis), ns.cumprod(x, axis=axis)]
    return outs, [x]


def case_cumsum_rows_f32(ns):
    x = _f32(np.random.RandomState(4).normal(0, 1, (6, 5000)))
    return [ns.cumsum(x, axis=1)], [x]


def case_cumprod_rows_f32(ns):
    x = _f32(np.random.RandomState(5).uniform(0.99, 1.01, (6, 5000)))
    return [ns.cumprod(x, axis=1)], [x]


def case_cumsum_rank1_f32(ns):
    x = _f32(np.random.RandomState(6).normal(0, 1, 20001))
    return [ns.cumsum(x)], [x]


def case_cumsum_axis0_f32(ns):
    x = _f32(np.random.RandomState(7).normal(0, 1, (300, 40)))
    return [ns.cumsum(x, axis=0)], [x]


def case_cumsum_int32(ns):
    x = np.random.RandomState(8).randint(-1000, 1000, (3, 4100)).astype(np.int32)
    return [ns.cumsum(x, axis=1)], [x]


def case_cumsum_f64(ns):
    x = np.random.RandomState(9).normal(0, 1, (2, 3000))
    return [ns.cumsum(x, axis=1)], [x]


def case_lstm_fwd(ns):
    rs = np.random.RandomState(20)
    g = _f32(rs.normal(0, 1, (6, 80)))
    c = _f32(rs.normal(0, 1, (6, 20)))
    op = ns.lstm(g, c, forget_bias=0.0)
    return [op[0], op[1]], [g, c]


def case_lstm_grad(ns):
    rs = np.random.RandomState(21)
    g = _f32(rs.normal(0, 1, (6, 80)))
    c = _f32(rs.normal(0, 1, (6, 20)))
    dc = _f32(rs.normal(0, 0.1, (6, 20)))
    dh = _f32(rs.normal(0, 0.1, (6, 20)))
    op = ns.lstm_grad(g, c, dc, dh, forget_bias=0.0)
    return [op[0], op[1]], [g, c, dc, dh]


def case_lstm_fwd_bias_odd(ns):
    rs = np.random.RandomState(22)
    g = _f32(rs.normal(0, 1, (3, 28)))
    c = _f32(rs.normal(0, 1, (3, 7)))
    op = ns.lstm(g, c, forget_bias=1.0)
    return [op[0], op[1]], [g, c]


def case_chain16(ns):
    x = _f32(np.random.RandomState(30).uniform(-2, 2, (3, 1000)))
    return [chain16(ns, x)], [x]


def case_chain16_light(ns):
    x = _f32(np.random.RandomState(35).uniform(-2, 2, (3, 1000)))
    return [chain16_light(ns, x)], [x]


def case_stdops_lstm(ns):
    rs = np.random.RandomState(31)
    g = _f32(rs.normal(0, 1, (4, 48)))
    c = _f32(rs.normal(0, 1, (4, 12)))
    return stdops_lstm(ns, g, c), [g, c]


def case_stdops_binary_f32(ns):
    so = ns.stdops
    rs = np.random.RandomState(32)
    a = _f32(rs.uniform(0.5, 2, (5, 8)))
    b = _f32(rs.uniform(0.5, 2, (5, 8)))
    s = _f32([1.5])
    return [so.add(a, b), so.sub(a, b), so.mul(a, b), so.div(a, b), so.mod(a, b), so.add(a, s), so.mul(s, b),
            so.less(a, b), so.greater_equal(a, b), so.equal(a, a), so.neg(a), so.sin(a), so.cos(a), so.tan(a)], \
        [a, b, s]


def case_stdops_int(ns):
    so = ns.stdops
    rs = np.random.RandomState(33)
    a = rs.randint(-50, 50, (4, 6)).astype(np.int32)
    b = rs.randint(1, 9, (4, 6)).astype(np.int32)
    return [so.add(a, b), so.sub(a, b), so.mul(a, b), so.div(a, b), so.mod(a, b), so.less_equal(a, b),
            so.not_equal(a, b), so.neg(a)], [a, b]


def case_stdops_concat_split(ns):
    so = ns.stdops
    rs = np.random.RandomState(34)
    a = _f32(rs.normal(size=(3, 4)))
    b = _f32(rs.normal(size=(3, 4)))
    c = _f32(rs.normal(size=(3, 6)))
    same = so.concat(a, b, concat_dim=1)
    ragged = so.concat(a, c, b, concat_dim=1)
    rows = so.concat(a, b, concat_dim=0)
    parts = so.split(same, split_dim=1, num_split=4)
    return [same, ragged, rows, parts[0], parts[3]], [a, b, c]


def _unary_case(ns, np_dtype, seed):
    ovl = ns.ovl
    fns = ['arccos', 'arcsin', 'arctan', 'cos', 'cosh', 'sin', 'sinh', 'tan', 'tanh', 'exp', 'log', 'log10', 'sqrt',
           'ceil', 'floor', 'absolute', 'isinf', 'isfinite', 'isnan', 'logical_not']

    @ovl.operator()
    def unary_all(x):
        pos = ovl.position_in(x.shape)
        outs = []
        for name in fns:
            out = ovl.output_like(x)
            out[pos] = getattr(ovl, name)(x[pos])
            outs.append(out)
        neg = ovl.output_like(x)
        neg[pos] = -x[pos]
        outs.append(neg)
        return outs

    x = np.random.RandomState(seed).uniform(0.01, 0.99, 37).astype(np_dtype)
    x[:4] = [0.5, 0.25, 0.75, 0.125]
    op = unary_all(x)
    return [op[i] for i in range(len(fns) + 1)], [x]


def case_unary_f32(ns):
    return _unary_case(ns, np.float32, 40)


def case_unary_f64(ns):
    return _unary_case(ns, np.float64, 41)


def _binary_case(ns, np_dtype, seed):
    ovl = ns.ovl
    is_float = np.dtype(np_dtype).kind == 'f'

    @ovl.operator()
    def binary_all(x, y):
        pos = ovl.position_in(x.shape)
        a, b = x[pos], y[pos]
        vals = [a + b, a - b, a * b, a / b, a % b, a == b, a != b, a < b, a <= b, a > b, a >= b,
                ovl.minimum(a, b), ovl.maximum(a, b), ovl.logical_and(a, b), ovl.logical_or(a, b), a + 3, 7 - b]
        if is_float:
            vals += [ovl.power(a, b), ovl.arctan2(a, b)]
        outs = []
        for v in vals:
            out = ovl.output_like(x)
            out[pos] = v
            outs.append(out)
        return outs

    rs = np.random.RandomState(seed)
    if is_float:
        x = rs.uniform(-4, 4, 33).astype(np_dtype)
        y = rs.uniform(0.5, 3, 33).astype(np_dtype)
    elif np.dtype(np_dtype).kind == 'u':
        x = rs.randint(0, 100, 33).astype(np_dtype)
        y = rs.randint(1, 10, 33).astype(np_dtype)
    else:
        x = rs.randint(-60, 60, 33).astype(np_dtype)
        y = rs.randint(1, 10, 33).astype(np_dtype)
        y[::3] *= -1
    x[0] = y[0]
    op = binary_all(x, y)
    return [op[i] for i in range(len(op.output_types))], [x, y]


def case_binary_f32(ns):
    return _binary_case(ns, np.float32, 50)


def case_binary_f64(ns):
    return _binary_case(ns, np.float64, 51)


def case_binary_i8(ns):
    return _binary_case(ns, np.int8, 52)


def case_binary_i16(ns):
    return _binary_case(ns, np.int16, 53)


def case_binary_i32(ns):
    return _binary_case(ns, np.int32, 54)


def case_binary_i64(ns):
    return _binary_case(ns, np.int64, 55)


def case_binary_u8(ns):
    return _binary_case(ns, np.uint8, 56)


def case_binary_u16(ns):
    return _binary_case(ns, np.uint16, 57)


def case_binary_u32(ns):
    return _binary_case(ns, np.uint32, 58)


def case_binary_u64(ns):
    return _binary_case(ns, np.uint64, 59)


def case_clip_limits_cast(ns):
    ovl = ns.ovl

    @ovl.operator()
    def clip(arg, lo=None, hi=None):
        out = ovl.output_like(arg)
        pos = ovl.position_in(arg.shape)
        v = ovl.variable(arg[pos], arg.dtype)
        with ovl.if_(v > hi):
            v <<= hi
        with ovl.elif_(v < lo):
            v <<= lo
        out[pos] = v
        return out

    @ovl.operator()
    def limits(arg):
        pos = ovl.position_in(arg.shape)
        a = ovl.output_like(arg)
        b = ovl.output_like(arg)
        c = ovl.output_like(arg)
        d = ovl.output(arg.shape, ovl.int32)
        a[pos] = ovl.min_value(arg.dtype) + arg[pos] * 0
        b[pos] = ovl.max_value(arg.dtype) + arg[pos] * 0
        c[pos] = ovl.epsilon(arg.dtype) * arg[pos]
        d[pos] = ovl.cast(arg[pos] * 10, ovl.int32)
        return a, b, c, d

    x = _f32(np.random.RandomState(60).uniform(-2, 2, (7, 9)))
    lim = limits(x)
    return [clip(x, lo=-1.0, hi=1.0), lim[0], lim[1], lim[2], lim[3]], [x]


def case_loops_locals(ns):
    ovl = ns.ovl

    @ovl.operator()
    def dot_rows(x, y):
        # one worker per row: fp64 accumulator over a runtime-independent trip count, reversed second loop
        rows, cols = x.shape
        pos = ovl.position_in(rows)
        out = ovl.output([rows], ovl.float64)
        rev = ovl.output([rows], x.dtype)
        acc = ovl.variable(0, ovl.float64)
        for i in ovl.arange(cols):
            acc <<= acc + ovl.cast(x[pos[0], i], ovl.float64) * ovl.cast(y[pos[0], i], ovl.float64)
        out[pos] = acc
        r = ovl.variable(0, x.dtype)
        for j in ovl.arange(cols - 1, -1, -2):
            r <<= r * 0.5 + x[pos[0], j]
        rev[pos] = r
        return out, rev

    @ovl.operator()
    def local_hist(x):
        # worker-local tensor: running sums of the row's elements by column parity
        rows, cols = x.shape
        pos = ovl.position_in(rows)
        out = ovl.output([rows, 2], x.dtype)
        acc = ovl.zeros([2], x.dtype)
        for i in ovl.arange(cols):
            acc[i % 2] = acc[i % 2] + x[pos[0], i]
        out[pos[0], 0] = acc[0]
        out[pos[0], 1] = acc[1]
        return out

    rs = np.random.RandomState(61)
    x = _f32(rs.normal(size=(9, 17)))
    y = _f32(rs.normal(size=(9, 17)))
    d = dot_rows(x, y)
    return [d[0], d[1], local_hist(x)], [x, y]


def case_merge_graph(ns):
    """split -> add/add -> mul -> concatenate graph of opveclib/test/test_operator_merge.py:183-224."""
    ovl = ns.ovl

    @ovl.operator()
    def split4(in0):
        n_col = in0.shape[1]
        col = ovl.position_in(n_col)
        rows = [ovl.output(n_col, in0.dtype) for _ in range(4)]
        for r in range(4):
            rows[r][col] = in0[r, col]
        return rows

    @ovl.operator()
    def stack3(op0, op1, op2):
        n_col = op0.shape[0]
        col = ovl.position_in(n_col)
        out = ovl.output([3, n_col], op0.dtype)
        out[0, col] = op0[col]
        out[1, col] = op1[col]
        out[2, col] = op2[col]
        return out

    u = user_ops(ns)
    in0 = np.random.RandomState(62).uniform(size=(4, 5))
    r = split4(in0)
    sum0 = u.ew_add(r[0], r[1])
    sum1 = u.ew_add(r[2], r[3])
    prod0 = u.ew_mul(sum0, sum1)
    return [stack3(sum0, prod0, sum1), sum0], [in0]


_cache = {}


def merge_ops(ns):
    """Operators of the reference's merge tests (opveclib/test/test_operator_merge.py:22-179): scans down the rows
    and along the columns with zero-seeded accumulators, a loop that overwrites its variable (so it is NOT a
    reduction), clamped padding through index variables, cropping."""
    key = ('merge', id(ns.ovl))
    if key in _cache:
        return _cache[key]
    ovl = ns.ovl

    @ovl.operator()
    def scan_down_rows(m):
        rows, cols = m.shape
        col = ovl.position_in(cols)
        acc = ovl.variable(0, m.dtype)
        out = ovl.output_like(m)
        for row in ovl.arange(rows):
            acc <<= acc + m[row, col]
            out[row, col] = acc
        return out

    @ovl.operator()
    def scan_along_cols(m):
        rows, cols = m.shape
        row = ovl.position_in(rows)
        acc = ovl.variable(0, m.dtype)
        out = ovl.output_like(m)
        for col in ovl.arange(cols):
            acc <<= acc + m[row, col]
            out[row, col] = acc
        return out

    @ovl.operator()
    def last_product(a, b):
        # every iteration overwrites the variable: the result is the LAST product, not a sum
        rows, cols, work = a.shape[0], b.shape[1], a.shape[1]
        pos = ovl.position_in([rows, cols])
        out = ovl.output([rows, cols], a.dtype)
        acc = ovl.variable(0, dtype=a.dtype)
        for k in ovl.arange(work):
            acc <<= a[pos[0], k] * b[k, pos[1]]
        out[pos[0], pos[1]] = acc
        return out

    @ovl.operator()
    def pad_clamped(m, n=None):
        rows_in, cols_in = m.shape
        out = ovl.output([rows_in + 2 * n, cols_in + 2 * n], m.dtype)
        pos = ovl.position_in([rows_in + 2 * n, cols_in + 2 * n])
        r = ovl.variable(pos[0], dtype=pos.dtype)
        c = ovl.variable(pos[1], dtype=pos.dtype)
        with ovl.if_(r < n):
            r <<= 0
        with ovl.elif_(r >= (rows_in + n)):
            r <<= rows_in - 1
        with ovl.else_():
            r <<= r - n
        with ovl.if_(c < n):
            c <<= 0
        with ovl.elif_(c >= (cols_in + n)):
            c <<= cols_in - 1
        with ovl.else_():
            c <<= c - n
        out[pos[0], pos[1]] = m[r, c]
        return out

    @ovl.operator()
    def crop(m, n=None):
        rows, cols = m.shape[0] - 2 * n, m.shape[1] - 2 * n
        pos = ovl.position_in([rows, cols])
        out = ovl.output([rows, cols], m.dtype)
        out[pos[0], pos[1]] = m[n + pos[0], n + pos[1]]
        return out

    @ovl.operator()
    def rows_of_four(m):
        cols = m.shape[1]
        col = ovl.position_in(cols)
        outs = [ovl.output(cols, m.dtype) for _ in range(4)]
        for r in range(4):
            outs[r][col] = m[r, col]
        return outs

    ops = types.SimpleNamespace(scan_down_rows=scan_down_rows, scan_along_cols=scan_along_cols, last_product=last_product,
                                pad_clamped=pad_clamped, crop=crop, rows_of_four=rows_of_four)
    _cache[key] = ops
    return ops


def case_merge_scan_nested(ns):
    x = np.random.RandomState(71).random_sample([3, 5])
    m = merge_ops(ns)
    return [m.scan_down_rows(m.scan_down_rows(x))], [x]


def case_merge_scan_rows_then_cols(ns):
    x = np.random.RandomState(72).random_sample([3, 3])
    m = merge_ops(ns)
    return [m.scan_along_cols(m.scan_down_rows(x))], [x]


def case_merge_product_then_scan(ns):
    rs = np.random.RandomState(73)
    a, b = rs.random_sample([3, 5]), rs.random_sample([5, 2])
    m = merge_ops(ns)
    return [m.scan_along_cols(m.last_product(a, b))], [a, b]


def case_merge_pad_crop(ns):
    x = np.random.RandomState(74).random_sample([3, 5])
    m = merge_ops(ns)
    return [m.crop(m.pad_clamped(x, n=2), n=2)], [x]


def case_merge_add_tree(ns):
    rs = np.random.RandomState(75)
    in0, in1, in2, in3 = [rs.random_sample([5]) for _ in range(4)]
    u = user_ops(ns)
    sum0 = u.ew_add(in1, in2)
    return [u.ew_add(in0, sum0), u.ew_add(in3, sum0)], [in0, in1, in2, in3]


def case_merge_product_split_adds(ns):
    x = np.random.RandomState(76).random_sample([4, 4])
    m, u = merge_ops(ns), user_ops(ns)
    s = m.rows_of_four(m.last_product(x, x))
    return [u.ew_add(s[0], s[1]), u.ew_add(s[2], s[3])], [x]


def case_dot_reference_test(ns):
    # the reference's own test: RandomState(1), uniform(-1, 1), 100 vectors of 10 elements
    rng = np.random.RandomState(1)
    x = rng.uniform(-1, 1, (100, 10))
    y = rng.uniform(-1, 1, (100, 10))
    return [user_ops(ns).dot(x, y)], [x, y]


def case_dot_f64_rows(ns):
    rs = np.random.RandomState(41)
    x = rs.uniform(-1, 1, (37, 1003))
    y = rs.uniform(-1, 1, (37, 1003))
    return [user_ops(ns).dot(x, y)], [x, y]


def case_matvec_doc(ns):
    # the documentation's example: [[0,1,2],[3,4,5],[6,7,8]] . [1,2,3] = [8, 26, 44]
    m = _f32([[0, 1, 2], [3, 4, 5], [6, 7, 8]])
    v = _f32([1, 2, 3])
    return [user_ops(ns).matvec(m, v)], [m, v]


def case_matvec_f32_long(ns):
    rs = np.random.RandomState(42)
    m = _f32(rs.uniform(-1, 1, (5, 9001)))
    v = _f32(rs.uniform(-1, 1, 9001))
    return [user_ops(ns).matvec(m, v)], [m, v]


def case_matvec_i32(ns):
    rs = np.random.RandomState(43)
    m = rs.randint(-1000, 1000, (19, 300)).astype(np.int32)
    v = rs.randint(-1000, 1000, 300).astype(np.int32)
    return [user_ops(ns).matvec(m, v)], [m, v]


def case_rowprod_scaled(ns):
    rs = np.random.RandomState(44)
    x = _f32(rs.uniform(0.99, 1.01, (3, 7, 500)))
    s = _f32(rs.uniform(0.5, 2, 7))
    return [user_ops(ns).rowprod_scaled(x, s)], [x, s]


def case_conv1d_same_nce(ns):
    rs = np.random.RandomState(51)
    x = _f32(rs.uniform(-1, 1, (2, 3, 37)))
    v = _f32(rs.uniform(-1, 1, (4, 3, 5)))
    return [ns.conv_1d(x, v, mode='same', kernel_orientation='as-is', data_format='NCE')], [x, v]


def case_conv1d_full_flipped_nec(ns):
    rs = np.random.RandomState(52)
    x = rs.uniform(-1, 1, (2, 29, 3))
    v = rs.uniform(-1, 1, (2, 4, 3))
    return [ns.conv_1d(x, v, mode='full', kernel_orientation='flipped', data_format='NEC')], [x, v]


def case_conv1d_valid_nce(ns):
    rs = np.random.RandomState(53)
    x = _f32(rs.uniform(-1, 1, (1, 2, 64)))
    v = _f32(rs.uniform(-1, 1, (3, 2, 7)))
    return [ns.conv_1d(x, v, mode='valid', kernel_orientation='as-is', data_format='NCE')], [x, v]


CASES = {name[len('case_'):]: fn for name, fn in sorted(globals().items()) if name.startswith('case_')}

# cases whose outputs involve libm transcendentals (compared with a tolerance on the GPU)
TRANSCENDENTAL = {'c1_chain', 'c1_chain_odd', 'expm1_f64', 'log1p_f64', 'lstm_fwd', 'lstm_grad', 'lstm_fwd_bias_odd',
                  'chain16', 'stdops_lstm', 'stdops_binary_f32', 'unary_f32', 'unary_f64', 'binary_f32', 'binary_f64'}
# cases that contain a re-associated scan on the GPU (compared with a scaled absolute tolerance)
SCANS = {'cumsum_rows_f32', 'cumprod_rows_f32', 'cumsum_rank1_f32', 'cumsum_f64', 'cumsum_axis0_f32'}
# axis along which those cases scan, where it is not the last one
SCAN_AXIS = {'cumsum_axis0_f32': 0}
# cases that contain a re-associated reduction loop on the GPU (floating point: compared with a tolerance)
REDUCTIONS = {'dot_f64_rows', 'matvec_f32_long', 'rowprod_scaled'}
