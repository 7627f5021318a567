"""The CUDA path against the REFERENCE-BUILT CPU operators (oracle/_ref: C++ emitted by the reference's own tracer,
merger and generator, compiled against its headers) at the sizes of the benchmark configurations, in both math lowerings.

exact       integer work and data movement bit-exact; transcendental chains within rtol 1e-5 (floor 1e-6 * max|ref|
            where the reference value comes from a cancellation) and at least 99.5 % of the elements inside the
            pure rtol; scans against the reference operator built and run in fp64 and cast to fp32.
tolerance   the same bounds - this lowering spends the tolerance on fewer instructions, it does not widen it.  The
            error statistics of every workload (largest relative error, distribution of the distance in ulps, share
            inside the pure rtol) are written to $OVL_TEST_REPORT_DIR/tolerance_math.json when that variable is set.

Skipped where oracle/_ref has not been built.
"""
import json
import os

import numpy as np
import pytest

import cases
from helpers import DRYRUN, assert_close, assert_exact
from oracle import ref_runner

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_runner.available(), reason='oracle/_ref has not been built')]

_report = {}


def _stats(got, want):
    g, w = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    ok = np.isfinite(w) & (w != 0)
    rel = np.abs(g - w)[ok] / np.abs(w[ok])
    ulp = np.abs(g - w)[ok] / np.spacing(np.abs(want.ravel()[ok]))
    return {'elements': int(ok.sum()), 'max_rel': float(rel.max()), 'max_abs': float(np.abs(g - w)[ok].max()),
            'inside_rtol_1e-5': float(np.mean(rel <= 1e-5)),
            'ulp_at_most': {str(k): float(np.mean(ulp <= k)) for k in (0, 1, 2, 4, 8, 16, 64)}}


def _check_transcendental(name, math, got, want):
    scale = float(np.abs(want[np.isfinite(want)]).max())
    assert_close(got, want, rtol=1e-5, atol=1e-6 * scale, what='%s (%s)' % (name, math))
    st = _stats(got, want)
    _report.setdefault(math, {})[name] = st
    assert st['inside_rtol_1e-5'] >= 0.995, '%s (%s): %r' % (name, math, st)


def _ref(name, ins):
    if not ref_runner.available(name):
        pytest.skip(name + ' is not in oracle/_ref')
    outs, _ = ref_runner.run(name, ins, num_threads=0, variant='opt', iterations=1)
    return outs


@pytest.fixture(scope='module', autouse=True)
def _write_report():
    yield
    where = os.environ.get('OVL_TEST_REPORT_DIR')
    if where and _report:
        os.makedirs(where, exist_ok=True)
        with open(os.path.join(where, 'tolerance_math.json'), 'w') as f:
            json.dump(_report, f, indent=1, sort_keys=True)


@pytest.mark.parametrize('math', ['exact', 'tolerance'])
def test_config1_chain_and_shift(math):
    ns = cases.impl()
    x = np.random.RandomState(1).uniform(-1, 1, 1 << 20).astype(np.float32)
    got_chain, got_shift = ns.ovl.evaluate([cases.c1_chain(ns, x), cases.user_ops(ns).shift_cyclic(x)], math=math)
    if DRYRUN:
        return          # (kernels compiled, nothing launched)
    assert_exact(got_shift, _ref('c1_shift_1048576', [x])[0], 'shift_cyclic 2^20 (%s)' % math)
    _check_transcendental('c1_chain', math, got_chain, _ref('c1_chain_1048576', [x])[0])


@pytest.mark.parametrize('math', ['exact', 'tolerance'])
def test_config3_lstm_forward_and_gradient(math):
    ns = cases.impl()
    rs = np.random.RandomState(3)
    g = rs.normal(0, 1, (512, 4096)).astype(np.float32)
    c = rs.normal(0, 1, (512, 1024)).astype(np.float32)
    dc = rs.normal(0, 0.1, (512, 1024)).astype(np.float32)
    dh = rs.normal(0, 0.1, (512, 1024)).astype(np.float32)
    fwd = ns.lstm(g, c, forget_bias=0.0)
    bwd = ns.lstm_grad(g, c, dc, dh, forget_bias=0.0)
    got = ns.ovl.evaluate([fwd[0], fwd[1], bwd[0], bwd[1]], math=math)
    if DRYRUN:
        return
    want = _ref('c3_lstm_512x1024', [g, c]) + _ref('c3_lstm_grad_512x1024', [g, c, dc, dh])
    for name, a, b in zip(('lstm_new_c', 'lstm_new_h', 'lstm_d_concat', 'lstm_d_c'), got, want):
        _check_transcendental(name, math, a, np.asarray(b).reshape(a.shape))


@pytest.mark.parametrize('math', ['exact', 'tolerance'])
def test_config4_slice(math):
    """One row slice [1, 2^24] of the sixteen-operator chain (the reference runs it as ten operators)."""
    ns = cases.impl()
    x = np.random.RandomState(1234).uniform(-2, 2, (1, 1 << 24)).astype(np.float32)
    got = ns.ovl.evaluate([cases.chain16(ns, x)], math=math)
    if DRYRUN:
        return
    want = np.asarray(_ref('c4_chain16_1x16777216', [x])[0]).reshape(got.shape)
    _check_transcendental('c4_chain16', math, got, want)


def test_tolerance_mode_leaves_integer_and_exact_arithmetic_alone():
    """Only fp32 division, exp, log and tanh change with the math lowering: a graph without them gives the same
    bits in both modes (packed additions and multiplications round like single ones), and so does integer work."""
    ns = cases.impl()
    x = np.random.RandomState(8).uniform(-2, 2, (4, 1 << 18)).astype(np.float32)
    a = ns.ovl.evaluate([cases.chain16_light(ns, x)], math='exact')
    b = ns.ovl.evaluate([cases.chain16_light(ns, x)], math='tolerance')
    i = np.random.RandomState(9).randint(-1000, 1000, (64, 64)).astype(np.int32)
    got_i = ns.ovl.evaluate([ns.cumsum(i, axis=1)], math='tolerance')
    if DRYRUN:
        return
    assert_exact(b, a, 'add / mul / where chain: tolerance vs exact')
    from opveclib_b200 import runtime
    prog, _ = runtime.compile_outputs([cases.chain16_light(ns, x)], math='tolerance')
    assert prog.plans[0].meta['vec']['paired'] and prog.plans[0].last_variant == 'vec'
    assert_exact(got_i, np.cumsum(i, axis=1, dtype=np.int32), 'int scan')


def test_packed_bodies_with_nested_and_partial_branches():
    """Branch shapes that the packed body cannot turn into one nested select - branches that assign several
    variables, nested chains, a chain without else, a store under a condition - are evaluated with per-worker masks.
    Exact arithmetic only, so the result must equal the exact lowering and the CPU oracle bit for bit."""
    from opveclib_b200 import runtime
    from oracle import runner
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def tangle(a, b):
        out = ovl.output_like(a)
        side = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        p = ovl.variable(0, a.dtype)
        q = ovl.variable(1, a.dtype)
        with ovl.if_(a[pos] > b[pos]):
            p <<= a[pos] - b[pos]
            q <<= a[pos] * 2.0
            with ovl.if_(a[pos] > 1.0):
                p <<= p + 0.25
            with ovl.elif_(b[pos] < -1.0):
                q <<= q - b[pos]
        with ovl.elif_(a[pos] < -0.5):
            p <<= b[pos] * b[pos]
        with ovl.if_(ovl.logical_or(p > 2.0, q < 0.0)):
            side[pos] = p * q
        with ovl.else_():
            side[pos] = ovl.minimum(p, q) - ovl.maximum(a[pos], b[pos])
        out[pos] = p + q * 0.5
        return out, side

    rs = np.random.RandomState(4)
    a = rs.uniform(-2, 2, (3, 4096)).astype(np.float32)
    b = rs.uniform(-2, 2, (3, 4096)).astype(np.float32)
    op = tangle(a, b)
    outs = [op[0], op[1]]
    exact = ns.ovl.evaluate(outs, math='exact')
    packed = ns.ovl.evaluate(outs, math='tolerance')
    prog, _ = runtime.compile_outputs(outs, math='tolerance')
    assert prog.plans[0].meta['vec']['paired']
    if DRYRUN:
        return
    want = runner.evaluate(outs)
    for k in range(2):
        assert_exact(exact[k], want[k], 'exact lowering output %d' % k)
        assert_exact(packed[k], want[k], 'packed body output %d' % k)


def test_tolerance_mode_special_values():
    """Zero, negative, infinite, NaN and subnormal arguments: log, exp, tanh and the division give what the exact
    functions give, except that subnormal arguments and results count as zero."""
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def probe(a, b):
        lg, ex, th, dv = ovl.output_like(a), ovl.output_like(a), ovl.output_like(a), ovl.output_like(a)
        l10, sq = ovl.output_like(a), ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        lg[pos] = ovl.log(a[pos])
        ex[pos] = ovl.exp(a[pos])
        th[pos] = ovl.tanh(a[pos])
        dv[pos] = a[pos] / b[pos]
        l10[pos] = ovl.log10(a[pos])
        sq[pos] = ovl.sqrt(a[pos])
        return lg, ex, th, dv, l10, sq

    inf, nan = np.inf, np.nan
    a = np.array([0.0, -0.0, 1.0, -1.0, inf, -inf, nan, 1e-30, 3e38, 88.0, -87.0, 100.0, -104.0, 20.0, -20.0, 0.5],
                 dtype=np.float32)
    b = np.array([1.0, 1.0, 0.0, inf, 1.0, 2.0, 1.0, 1e30, 1e-30, nan, -0.0, inf, -inf, 3.0, 7.0, 0.0], dtype=np.float32)
    op = probe(a, b)
    got = ovl.evaluate([op[0], op[1], op[2], op[3], op[4], op[5]], math='tolerance')
    if DRYRUN:
        return
    with np.errstate(all='ignore'):
        want = [np.log(a), np.exp(a), np.tanh(a), a / b, np.log10(a), np.sqrt(a)]
    for name, g, w in zip(('log', 'exp', 'tanh', 'div', 'log10', 'sqrt'), got, want):
        w = w.astype(np.float32)
        assert np.array_equal(np.isnan(g), np.isnan(w)), name
        fin = np.isfinite(w) & (np.abs(w) >= 1.2e-38)
        assert np.array_equal(g[~np.isfinite(w) & ~np.isnan(w)], w[~np.isfinite(w) & ~np.isnan(w)]), name
        np.testing.assert_allclose(g[fin], w[fin], rtol=1e-5, err_msg=name)
        tiny = ~np.isnan(w) & (np.abs(w) < 1.2e-38)
        assert np.all(np.abs(g[tiny]) < 1.2e-38), name


def test_operator_library_lstm_is_one_vectorised_kernel():
    """The LSTM cell composed from the operator library (split, sigmoid, tanh, mul, add: the graph of
    opveclib/test/test_operator_merge.py:311-321) at the size of benchmark configuration 3 fuses into ONE kernel that takes the
    vectorised path - the hand-fused cell's kernel shape - and agrees with the CPU oracle."""
    from opveclib_b200 import runtime
    from oracle import runner
    ns = cases.impl()
    rs = np.random.RandomState(13)
    g = rs.normal(0, 1, (512, 4096)).astype(np.float32)
    c = rs.normal(0, 1, (512, 1024)).astype(np.float32)
    for math in ('exact', 'tolerance'):
        outs = cases.stdops_lstm(ns, g, c)
        got = ns.ovl.evaluate(outs, math=math)
        prog, _ = runtime.compile_outputs(outs, math=math)
        assert len(prog.plans) == 1 and prog.plans[0].meta['vec'] is not None
        assert prog.plans[0].meta['vec']['lanes'] == 4
        if DRYRUN:
            continue
        assert prog.plans[0].last_variant == 'vec'
        want = runner.evaluate(outs)
        for name, a, b in zip(('new_c', 'new_h'), got, want):
            _check_transcendental('stdops_lstm_' + name, math, a, b)


def test_config2_sampled_rows():
    ns = cases.impl()
    rs = np.random.RandomState(2)
    for op, name, x in ((ns.cumsum, 'c2_cumsum_4096x8192', rs.normal(0, 1, (4096, 8192)).astype(np.float32)),
                        (ns.cumprod, 'c2_cumprod_4096x8192', rs.uniform(0.99, 1.01, (4096, 8192)).astype(np.float32))):
        got = ns.ovl.evaluate([op(x, axis=1)])
        if DRYRUN:
            continue
        want = np.asarray(_ref(name, [x])[0]).reshape(got.shape)
        rows = [0, 1, 2047, 4095] + list(np.random.RandomState(5).randint(0, 4096, 28))
        # the reference adds serially in fp32, the GPU scan accumulates in fp64: they differ by the reference's own
        # accumulated rounding
        line_max = np.abs(want[rows].astype(np.float64)).max(axis=1, keepdims=True)
        assert_close(got[rows], want[rows], rtol=1e-5, atol=1e-5 * line_max * np.ones(want[rows].shape), what=name)


def test_config5_prefix_against_the_reference_operator_run_in_fp64():
    """The first 2^26 elements of the scan against the reference's own cumsum operator traced for fp64 input, run on
    the host and cast to fp32: rtol 1e-5, and in fact the exact scan rounded once."""
    if DRYRUN:
        pytest.skip('needs a device')
    import torch
    from opveclib_b200 import parallel
    n = 1 << 26
    x = np.random.RandomState(5).normal(0, 1, n).astype(np.float32)
    want64 = np.asarray(_ref('c5_cumsum_f64_%d' % n, [x.astype(np.float64)])[0]).reshape(-1)
    scan = parallel.ShardedScan(n, 'add')
    got = scan(torch.from_numpy(x).cuda()).cpu().numpy()
    scan.check_status()
    err = np.abs(got.astype(np.float64) - want64)
    # the serial fp64 loop itself carries rounding of about 1e-16 * sqrt(n) * |partial sums|: an absolute floor far
    # below an fp32 ulp of the values that occur
    assert np.all(err <= 1e-5 * np.abs(want64) + 1e-6)
    assert np.all(err <= 6.0e-8 * np.abs(want64) + 1e-6)
