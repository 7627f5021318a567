"""Scans along an axis that is not the contiguous one: a block walks down all rows of a strip of columns (one
launch) when there is a strip per SM, else warps walk down chunks of rows in three passes.

Checked against numpy (fp64 accumulation for floating-point data, wrapping integer arithmetic otherwise) on shapes
with ragged row chunks, ragged column strips, several outer slabs, and on the shape of the reference's own timing
harness (opveclib/examples/test_perf_accumulate.py:35-48: fp64 [10000, 1000] along axis 0)."""
import numpy as np
import pytest

import cases
from helpers import DRYRUN

pytestmark = pytest.mark.gpu

SHAPES = [((1000, 200), 0, 'float64'), ((300, 7, 33), 0, 'float32'), ((5, 400, 64), 1, 'float32'),
          ((2000, 33), 0, 'int32'), ((257, 128), 0, 'float32'), ((3, 1000, 4), 1, 'float64'), ((4096, 64), 0, 'float32'),
          ((700, 3, 5), 0, 'uint8')]
# enough columns for the one-launch walk: ragged last strips, ragged last tiles, narrow strips (8 and 4 columns),
# several outer slabs, an integer type
WALK_SHAPES = [((1000, 5000), 0, 'float32', 32), ((300, 1201), 0, 'float64', 8), ((3, 500, 2000), 1, 'int32', 32),
               ((2100, 601), 0, 'float64', 4), ((261, 4800), 0, 'float32', 32), ((6, 3000, 200), 1, 'float32', 8)]


def _reference(x, fn, axis):
    if x.dtype.kind == 'f':
        wide = x.astype(np.float64)
        return (np.cumsum(wide, axis=axis) if fn == 'cumsum' else np.cumprod(wide, axis=axis)).astype(x.dtype)
    return np.cumsum(x, axis=axis, dtype=x.dtype) if fn == 'cumsum' else np.cumprod(x, axis=axis, dtype=x.dtype)


@pytest.mark.parametrize('fn', ['cumsum', 'cumprod'])
@pytest.mark.parametrize('shape,axis,dtype', SHAPES)
def test_scan_along_a_strided_axis(shape, axis, dtype, fn):
    from opveclib_b200 import runtime
    ns = cases.impl()
    rs = np.random.RandomState(len(shape) * 7 + axis)
    if dtype.startswith('float'):
        x = (rs.normal(0, 1, shape) if fn == 'cumsum' else rs.uniform(0.999, 1.001, shape)).astype(dtype)
    else:
        x = rs.randint(0, 3, shape).astype(dtype)
    op = getattr(ns, fn)(x, axis=axis)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    plan = prog.plans[0]
    assert plan.meta['scan'] is not None and plan.meta['scan']['strided']
    if DRYRUN:
        return
    assert plan.last_variant in ('cscan', 'cscanu')
    want = _reference(x, fn, axis)
    if dtype == 'float32':
        np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)
    elif dtype == 'float64':
        np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-10)
    else:
        np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize('fn', ['cumsum', 'cumprod'])
@pytest.mark.parametrize('shape,axis,dtype,width', WALK_SHAPES)
def test_one_launch_walk_down_strips_of_columns(shape, axis, dtype, width, fn):
    from opveclib_b200 import runtime
    ns = cases.impl()
    rs = np.random.RandomState(sum(shape) + axis)
    if dtype.startswith('float'):
        x = (rs.normal(0, 1, shape) if fn == 'cumsum' else rs.uniform(0.999, 1.001, shape)).astype(dtype)
    else:
        x = rs.randint(-2, 3, shape).astype(dtype)
    op = getattr(ns, fn)(x, axis=axis)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    plan = prog.plans[0]
    assert plan.meta['scan']['walk'] is not None and plan.meta['scan']['walk']['width'] == width
    if DRYRUN:
        return
    assert plan.last_variant == 'cwalk'
    want = _reference(x, fn, axis)
    if dtype == 'float32':
        np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)
    elif dtype == 'float64':
        np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-10)
    else:
        np.testing.assert_array_equal(got, want)


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_unaligned_device_tensor_uses_the_scalar_variant():
    import torch
    from opveclib_b200 import runtime
    ns = cases.impl()
    x = np.random.RandomState(3).normal(0, 1, (600, 64)).astype(np.float32)
    base = torch.empty(600 * 64 + 1, dtype=torch.float32, device='cuda')
    dx = base[1:].view(600, 64)
    dx.copy_(torch.from_numpy(x))
    assert dx.data_ptr() % 16 != 0
    op = ns.cumsum(dx, axis=0)
    got = ns.ovl.evaluate([op]).cpu().numpy()
    prog, _ = runtime.compile_outputs([op])
    assert prog.plans[0].meta['scan']['walk'] is None and prog.plans[0].last_variant == 'cscanu'
    np.testing.assert_allclose(got, _reference(x, 'cumsum', 0), rtol=1.3e-7, atol=0)


def test_the_reference_timing_harness_shape():
    ns = cases.impl()
    x = np.random.RandomState(1).uniform(0, 1, size=(10000, 1000))
    got = ns.ovl.evaluate(ns.cumsum(x, axis=0))
    if not DRYRUN:
        assert np.allclose(np.cumsum(x, axis=0), got)          # the harness's own check
        np.testing.assert_allclose(got, np.cumsum(x, axis=0), rtol=1e-12, atol=1e-9)


def test_profile_with_several_iterations_returns_the_scan():
    """The reference's timing harness calls ``ovl.profile(cumsum(x, axis=0), profiling_iterations=10)`` and
    checks the result (opveclib/examples/test_perf_accumulate.py:50-53).  Multi-pass scans must run one whole
    pass sequence per timed iteration: their middle pass rewrites the tile aggregates in place."""
    ns = cases.impl()
    x = np.random.RandomState(2).uniform(0, 1, size=(10000, 1000))
    outs, times = ns.ovl.profile(ns.cumsum(x, axis=0), profiling_iterations=3)
    if not DRYRUN:
        np.testing.assert_allclose(outs[0], np.cumsum(x, axis=0), rtol=1e-12, atol=1e-9)
        assert all(len(ms) == 3 and np.all(ms > 0) for ms in times.values())


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_profile_with_several_iterations_on_an_unaligned_long_line():
    """Three-pass contiguous scan (a long line that does not start on a 16-byte boundary), three timed iterations."""
    import torch
    ns = cases.impl()
    n = 3 * 8192 * 5 + 77
    x = np.random.RandomState(4).normal(0, 1, n).astype(np.float32)
    base = torch.empty(n + 1, dtype=torch.float32, device='cuda')
    dx = base[1:]
    dx.copy_(torch.from_numpy(x))
    assert dx.data_ptr() % 16 != 0
    outs, times = ns.ovl.profile(ns.cumsum(dx), profiling_iterations=3)
    want = np.cumsum(x.astype(np.float64))
    np.testing.assert_allclose(outs[0].cpu().numpy(), want, rtol=1e-5, atol=1e-5 * np.abs(want).max())
    assert all(len(ms) == 3 for ms in times.values())
