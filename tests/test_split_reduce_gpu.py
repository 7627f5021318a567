"""Reduction loops of few workers and many trips: the loop of a worker (or of 32 neighbouring workers) is cut into
slices that different thread blocks fold; the block that delivers the last slice combines them in slice order.
Integer results must equal the serial loop bit for bit, floating-point ones within the reordering bound, and a
repeated launch must give the same bits."""
import numpy as np
import pytest

import cases
from helpers import DRYRUN

pytestmark = pytest.mark.gpu


def _run(ns, outputs, **kw):
    got = ns.ovl.evaluate(outputs, target_language='b200', **kw)
    if DRYRUN:
        pytest.skip('compiled; needs a device to run')
    return got


def _plan(ns, outputs):
    from opveclib_b200 import runtime
    prog, _ = runtime.compile_outputs(outputs)
    return prog.plans[0]


@pytest.mark.parametrize('rows,cols', [(1, 1 << 22), (3, 1 << 20), (5, (1 << 18) + 77)])
def test_split_matvec_fp32(rows, cols):
    ns = cases.impl()
    rs = np.random.RandomState(rows)
    m = rs.uniform(-1, 1, (rows, cols)).astype(np.float32)
    v = rs.uniform(-1, 1, cols).astype(np.float32)
    op = [cases.user_ops(ns).matvec(m, v)]
    assert _plan(ns, op).meta['red'].get('split')
    got = _run(ns, op)
    assert _plan(ns, op).last_variant == 'red'
    prod = m.astype(np.float64) * v.astype(np.float64)
    want = prod.sum(axis=1)
    # fp32 accumulation in a fixed tree: the error is bounded by eps * sum |terms| times the depth of the partial sums
    bound = 2e-5 * np.abs(prod).sum(axis=1)
    assert np.all(np.abs(got.astype(np.float64) - want) <= bound)
    again = _run(ns, op)
    assert np.array_equal(got, again)


def test_split_dot_fp64_matches_a_pairwise_sum():
    ns = cases.impl()
    rs = np.random.RandomState(7)
    a = rs.normal(0, 1, (2, 1 << 20))
    b = rs.normal(0, 1, (2, 1 << 20))
    op = [cases.user_ops(ns).dot(a, b)]
    assert _plan(ns, op).meta['red'].get('split')
    got = _run(ns, op)
    want = np.array([np.sum(a[i] * b[i]) for i in range(2)])
    assert np.all(np.abs(got - want) <= 1e-12 * np.sum(np.abs(a * b), axis=1))


def test_split_matvec_int32_is_exact():
    ns = cases.impl()
    rs = np.random.RandomState(3)
    m = rs.randint(-1000, 1000, (2, 1 << 19)).astype(np.int32)
    v = rs.randint(-1000, 1000, 1 << 19).astype(np.int32)
    op = [cases.user_ops(ns).matvec(m, v)]
    assert _plan(ns, op).meta['red'].get('split')
    got = _run(ns, op)
    want = (m.astype(np.int64) * v.astype(np.int64)).sum(axis=1).astype(np.int32)      # wraps like int32 arithmetic
    assert np.array_equal(got, want)


@pytest.mark.parametrize('rows,cols,dtype', [(1 << 17, 48, np.float32), ((1 << 16) + 5, 16, np.float32),
                                             (1 << 16, 96, np.int32), (1 << 15, 8, np.float64)])
def test_split_column_sums(rows, cols, dtype):
    ns = cases.impl()
    rs = np.random.RandomState(cols)
    a = (rs.randint(-50, 50, (rows, cols)) if dtype == np.int32 else rs.normal(0, 1, (rows, cols))).astype(dtype)
    op = [cases.user_ops(ns).colsum(a)]
    red = _plan(ns, op).meta['red']
    assert red['layout'] == 'across' and red.get('split')
    got = _run(ns, op)
    assert _plan(ns, op).last_variant == 'red'
    if dtype == np.int32:
        assert np.array_equal(got, a.sum(axis=0, dtype=np.int64).astype(np.int32))
    else:
        eps = 2e-5 if dtype == np.float32 else 1e-12
        want = a.astype(np.float64).sum(axis=0)
        assert np.all(np.abs(got.astype(np.float64) - want) <= eps * np.abs(a.astype(np.float64)).sum(axis=0))
    assert np.array_equal(got, _run(ns, op))


def test_split_product_with_statements_after_the_loop():
    ns = cases.impl()
    rs = np.random.RandomState(11)
    # (factors spread around 1 on a log scale: factors within 1e-4 of 1 would make every fp32 product drop its
    # second-order term the same way, and the serial loop and the tree would drift apart by 5e-4)
    x = np.exp(rs.uniform(-0.1, 0.1, (2, 3, 1 << 16))).astype(np.float32)
    s = rs.uniform(1, 2, 3).astype(np.float32)
    op = [cases.user_ops(ns).rowprod_scaled(x, s)]
    assert _plan(ns, op).meta['red'].get('split')
    got = _run(ns, op)
    exact = np.prod(x.astype(np.float64), axis=2) * s.astype(np.float64)
    np.testing.assert_allclose(got, exact, rtol=5e-5)
    from oracle import runner
    np.testing.assert_allclose(got, runner.evaluate(op), rtol=1e-4)


def test_split_reduction_profiled_repeatedly_and_from_device_tensors():
    import torch
    ns = cases.impl()
    rs = np.random.RandomState(5)
    m = rs.uniform(-1, 1, (2, 1 << 20)).astype(np.float32)
    v = rs.uniform(-1, 1, 1 << 20).astype(np.float32)
    op = [cases.user_ops(ns).matvec(m, v)]
    once = _run(ns, op)
    outs, times = ns.ovl.profile(op, target_language='b200', profiling_iterations=4)
    assert np.array_equal(outs[0], once)          # the counters are cleared before every launch
    assert all(len(t) == 4 for t in times.values())
    md, vd = torch.from_numpy(m).cuda(), torch.from_numpy(v).cuda()
    got = ns.ovl.evaluate([cases.user_ops(ns).matvec(md, vd)], target_language='b200')
    assert np.array_equal(got.cpu().numpy(), once)


def _pool(ovl):
    @ovl.operator()
    def pool(x):
        # sum over the last two axes with a nest of two loops (global pooling of an image per batch and channel)
        out = ovl.output([x.shape[0], x.shape[1]], x.dtype)
        pos = ovl.position_in([x.shape[0], x.shape[1]])
        acc = ovl.variable(0, x.dtype)
        for i in ovl.arange(x.shape[2]):
            for j in ovl.arange(x.shape[3]):
                acc <<= acc + x[pos[0], pos[1], i, j]
        out[pos] = acc
        return out
    return pool


@pytest.mark.parametrize('shape,dtype', [((8, 64, 56, 56), np.float32), ((3, 5, 20, 30), np.int32),
                                         ((2, 1, 512, 512), np.float32), ((1, 3, 300, 301), np.int64)])
def test_nest_of_two_loops_is_reduced_as_one_loop(shape, dtype):
    """``for i: for j: acc += x[n, c, i, j]``: one loop over the pairs (i, j); with few workers and many trips the
    trips are also cut into slices for many blocks."""
    ns = cases.impl()
    rs = np.random.RandomState(shape[2])
    x = (rs.randint(-1000, 1000, shape) if np.dtype(dtype).kind == 'i' else rs.normal(0, 1, shape)).astype(dtype)
    op = [_pool(ns.ovl)(x)]
    red = _plan(ns, op).meta['red']
    assert red is not None and red['trips'] == shape[2] * shape[3]
    assert bool(red.get('split')) == (shape[2] * shape[3] >= 65536)
    got = _run(ns, op)
    assert _plan(ns, op).last_variant == 'red'
    if np.dtype(dtype).kind == 'i':
        assert np.array_equal(got, x.sum(axis=(2, 3), dtype=dtype))
    else:
        want = x.astype(np.float64).sum(axis=(2, 3))
        assert np.all(np.abs(got.astype(np.float64) - want) <= 2e-5 * np.abs(x.astype(np.float64)).sum(axis=(2, 3)))
    from oracle import runner
    np.testing.assert_allclose(got, runner.evaluate(op), rtol=1e-4, atol=1e-3)
