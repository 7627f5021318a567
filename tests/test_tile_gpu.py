"""Operands read along another axis than the innermost one of the workgroup (transposes and their fusions):
the `_tile` kernel stages them through shared memory, 32 x 32 workers at a time.  Results must equal the oracle's
bit for bit (data movement and exactly rounded arithmetic only)."""
import numpy as np
import pytest

import cases
from helpers import DRYRUN, assert_exact

pytestmark = pytest.mark.gpu


def _ops(ovl):
    @ovl.operator()
    def batched_transpose(a):
        out = ovl.output([a.shape[0], a.shape[2], a.shape[1]], a.dtype)
        pos = ovl.position_in(out.shape)
        out[pos] = a[pos[0], pos[2], pos[1]]
        return out

    @ovl.operator()
    def symmetrise(a):
        # the same operand both ways, and a branch on the transposed value
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        mirrored = a[pos[1], pos[0]]
        with ovl.if_(mirrored > a[pos]):
            out[pos] = mirrored
        with ovl.else_():
            out[pos] = a[pos] - mirrored
        return out

    @ovl.operator()
    def outer_to_inner(a):
        # [n, rows, cols] -> [rows, cols, n]: the operand is contiguous along the output's middle axis
        out = ovl.output([a.shape[1], a.shape[2], a.shape[0]], a.dtype)
        pos = ovl.position_in(out.shape)
        out[pos] = a[pos[2], pos[0], pos[1]]
        return out

    @ovl.operator()
    def scatter_transpose(a, scale=None):
        # the workgroup follows the operand; the result is written transposed
        out = ovl.output([a.shape[1], a.shape[0]], a.dtype)
        pos = ovl.position_in(a.shape)
        out[pos[1], pos[0]] = a[pos] * scale
        return out

    @ovl.operator()
    def both_ways(a, b):
        # b is read and the first result written along the workgroup's first axis; the second result goes straight
        flipped = ovl.output([a.shape[1], a.shape[0]], a.dtype)
        straight = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        total = a[pos] + b[pos[1], pos[0]]
        flipped[pos[1], pos[0]] = total
        straight[pos] = total - a[pos]
        return flipped, straight

    return batched_transpose, symmetrise, outer_to_inner, scatter_transpose, both_ways


_cache = {}


def ops(ns):
    if id(ns.ovl) not in _cache:
        _cache[id(ns.ovl)] = _ops(ns.ovl)
    return _cache[id(ns.ovl)]


def _check(ns, outs, expect_tile=True):
    from opveclib_b200 import runtime
    from oracle import runner
    got = ns.ovl.evaluate(outs)
    prog, _ = runtime.compile_outputs(outs)
    tiled = [p for p in prog.plans if p.meta.get('tile')]
    assert bool(tiled) == expect_tile
    if DRYRUN:
        return
    assert all(p.last_variant == 'tile' for p in tiled)
    want = runner.evaluate(outs)
    if len(outs) == 1:
        got, want = [got], [want]
    for g, w in zip(got, want):
        assert_exact(np.asarray(g), w, 'tile kernel')


@pytest.mark.parametrize('shape,dtype', [((64, 96), 'float32'), ((100, 37), 'float32'), ((33, 1000), 'float64'),
                                         ((257, 129), 'int16'), ((1024, 2048), 'float32'), ((32, 32), 'uint8')])
def test_transpose(shape, dtype):
    ns = cases.impl()
    transpose = cases.user_ops(ns).transpose
    rs = np.random.RandomState(shape[0])
    x = (rs.uniform(-4, 4, shape) if dtype.startswith('float') else rs.randint(0, 100, shape)).astype(dtype)
    out = transpose(x)
    _check(ns, [out])
    if not DRYRUN:
        assert_exact(np.asarray(ns.ovl.evaluate([out])), np.ascontiguousarray(x.T), 'against numpy')


def test_transposed_operand_fused_with_a_straight_one():
    ns = cases.impl()
    _, symmetrise, _, _, _ = ops(ns)
    transpose_axpy = cases.user_ops(ns).transpose_axpy
    rs = np.random.RandomState(5)
    a = rs.uniform(-1, 1, (300, 200)).astype(np.float32)
    b = rs.uniform(-1, 1, (200, 300)).astype(np.float32)
    _check(ns, [transpose_axpy(a, b, alpha=0.5)])
    sq = rs.uniform(-1, 1, (150, 150)).astype(np.float32)
    _check(ns, [symmetrise(sq)])
    # the staged kernel after fusion with element-wise neighbours
    u = cases.user_ops(ns)
    _check(ns, [u.ew_mulc(transpose_axpy(u.ew_addc(a, c=1.0), b, alpha=2.0), c=0.25)])


def test_rank_three_tiles_over_the_right_axes():
    ns = cases.impl()
    batched_transpose, _, outer_to_inner, _, _ = ops(ns)
    rs = np.random.RandomState(6)
    x = rs.uniform(-1, 1, (3, 70, 45)).astype(np.float32)
    _check(ns, [batched_transpose(x)])
    y = rs.randint(-50, 50, (40, 5, 64)).astype(np.int32)
    _check(ns, [outer_to_inner(y)])


def test_results_written_along_another_axis():
    ns = cases.impl()
    _, _, _, scatter_transpose, both_ways = ops(ns)
    rs = np.random.RandomState(7)
    for shape in ((64, 64), (130, 75), (40, 1000)):
        a = rs.uniform(-1, 1, shape).astype(np.float32)
        _check(ns, [scatter_transpose(a, scale=2.0)])
        if not DRYRUN:
            assert_exact(np.asarray(ns.ovl.evaluate([scatter_transpose(a, scale=2.0)])), np.ascontiguousarray(a.T * 2), 'numpy')
    a = rs.randint(-9, 9, (96, 200)).astype(np.int32)
    b = rs.randint(-9, 9, (200, 96)).astype(np.int32)
    op = both_ways(a, b)
    _check(ns, [op[0], op[1]])


def test_many_wide_operands_fall_back_to_narrower_tiles():
    """Three transposed fp64 operands do not fit in shared memory as 64 x 64 tiles; all three are still staged."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def three_transposed(a, b, c):
        out = ovl.output([a.shape[1], a.shape[0]], a.dtype)
        pos = ovl.position_in(out.shape)
        out[pos] = a[pos[1], pos[0]] * b[pos[1], pos[0]] - c[pos[1], pos[0]]
        return out

    rs = np.random.RandomState(8)
    a, b, c = (rs.uniform(-1, 1, (130, 200)) for _ in range(3))
    op = three_transposed(a, b, c)
    prog, _ = runtime.compile_outputs([op])
    assert prog.plans[0].meta['tile']['staged'] == 3
    _check(ns, [op])


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_staged_and_unstaged_kernels_agree(monkeypatch):
    """OVL_TILE_MODE=off runs the same graph through the vectorised kernel (operand read in place)."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    u = cases.user_ops(ns)
    rs = np.random.RandomState(12)
    a = rs.uniform(-1, 1, (500, 333)).astype(np.float32)
    b = rs.uniform(-1, 1, (333, 500)).astype(np.float32)
    op = u.transpose_axpy(a, b, alpha=0.75)
    staged = np.asarray(ns.ovl.evaluate([op]))
    prog, _ = runtime.compile_outputs([op])
    assert prog.plans[0].last_variant == 'tile'
    monkeypatch.setenv('OVL_TILE_MODE', 'off')
    plain = np.asarray(ns.ovl.evaluate([op]))
    assert prog.plans[0].last_variant in ('vec', 'gen')
    assert_exact(staged, plain, 'staged against unstaged')
    assert_exact(staged, (a.T * np.float32(0.75) + b).astype(np.float32), 'against numpy')


@pytest.mark.parametrize('shape,dtype', [((4096, 512), 'float32'), ((1000, 100), 'float64'), ((777, 45), 'int32'),
                                         ((130, 8192), 'float32')])
def test_column_sums_walk_the_rows_with_neighbouring_workers_on_a_warp(shape, dtype):
    from opveclib_b200 import runtime
    ns = cases.impl()
    rs = np.random.RandomState(shape[1])
    x = (rs.normal(0, 1, shape) if dtype.startswith('float') else rs.randint(-5, 6, shape)).astype(dtype)
    op = cases.user_ops(ns).colsum(x)
    got = np.asarray(ns.ovl.evaluate([op]))
    prog, _ = runtime.compile_outputs([op])
    assert prog.plans[0].meta['red']['layout'] == 'across'
    if DRYRUN:
        return
    assert prog.plans[0].last_variant == 'red'
    if dtype == 'int32':
        np.testing.assert_array_equal(got, x.sum(axis=0, dtype=np.int32))
    else:
        wide = x.astype(np.float64).sum(axis=0)
        scale = np.abs(x.astype(np.float64)).sum(axis=0)
        tol = 1e-5 if dtype == 'float32' else 1e-12
        assert np.all(np.abs(got - wide) <= tol * scale)


def test_weighted_column_sums_share_the_weights_across_the_warp():
    """`acc += a[i, col] * w[i]`: the weight is the same for every worker, the matrix decides the layout."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def weighted_colsum(a, w):
        out = ovl.output([a.shape[1]], a.dtype)
        col = ovl.position_in([a.shape[1]])[0]
        accum = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[0]):
            accum <<= accum + a[i, col] * w[i]
        out[col] = accum
        return out

    rs = np.random.RandomState(21)
    a, w = rs.normal(0, 1, (2000, 300)), rs.normal(0, 1, 2000)
    op = weighted_colsum(a, w)
    got = np.asarray(ns.ovl.evaluate([op]))
    prog, _ = runtime.compile_outputs([op])
    assert prog.plans[0].meta['red']['layout'] == 'across'
    if DRYRUN:
        return
    np.testing.assert_allclose(got, (a * w[:, None]).sum(axis=0), rtol=1e-11, atol=1e-11)


def test_small_or_straight_kernels_are_left_alone():
    ns = cases.impl()
    transpose = cases.user_ops(ns).transpose
    x = np.arange(6 * 8, dtype=np.float32).reshape(6, 8)
    _check(ns, [transpose(x)], expect_tile=False)        # narrower than a tile
    u = cases.user_ops(ns)
    _check(ns, [u.ew_mulc(np.ones((64, 64), np.float32), c=2.0)], expect_tile=False)
