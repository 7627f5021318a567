"""Scans of thousands of lines: one warp per line (`scan_lines_warp`), through generated kernels and through the
built-in fp32 entry point.  Checked against the exact scan computed in fp64 (or wrapping integer arithmetic)."""
import ctypes

import numpy as np
import pytest

import cases
from helpers import DRYRUN
from opveclib_b200 import launcher

pytestmark = pytest.mark.gpu

SHAPES = [((2048, 512), 'float32'), ((4096, 400), 'float32'), ((3000, 8192), 'float32'), ((2048, 68), 'int32'),
          ((2100, 1026), 'float64'), ((2500, 20004), 'float32'), ((2, 1100, 260), 'float32'), ((4096, 256), 'int16')]


def _reference(x, fn):
    axis = x.ndim - 1
    if x.dtype.kind == 'f':
        wide = x.astype(np.float64)
        return (np.cumsum(wide, axis=axis) if fn == 'cumsum' else np.cumprod(wide, axis=axis)).astype(x.dtype)
    return np.cumsum(x, axis=axis, dtype=x.dtype) if fn == 'cumsum' else np.cumprod(x, axis=axis, dtype=x.dtype)


@pytest.mark.parametrize('fn', ['cumsum', 'cumprod'])
@pytest.mark.parametrize('shape,dtype', SHAPES)
def test_generated_kernel_scans_a_line_per_warp(shape, dtype, fn):
    from opveclib_b200 import runtime
    ns = cases.impl()
    rs = np.random.RandomState(shape[-1])
    if dtype.startswith('float'):
        x = (rs.normal(0, 1, shape) if fn == 'cumsum' else rs.uniform(0.999, 1.001, shape)).astype(dtype)
    else:
        x = rs.randint(-2, 3, shape).astype(dtype)
    op = getattr(ns, fn)(x, axis=len(shape) - 1)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    plan = prog.plans[0]
    assert plan.meta['scan'] is not None and plan.meta['scan']['warp'] is not None
    if DRYRUN:
        return
    assert plan.last_variant == 'wscan'
    want = _reference(x, fn)
    if dtype == 'float32':
        np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)
    elif dtype == 'float64':
        np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-10)
    else:
        np.testing.assert_array_equal(got, want)


def test_fewer_lines_or_unaligned_lines_keep_the_block_kernels():
    from opveclib_b200 import runtime
    ns = cases.impl()
    for shape in ((100, 8192), (4096, 1025)):
        op = ns.cumsum(np.zeros(shape, np.float32), axis=1)
        prog, _ = runtime.compile_outputs([op])
        assert prog.plans[0].meta['scan']['warp'] is None


@pytest.mark.skipif(DRYRUN, reason='needs a device')
@pytest.mark.parametrize('op', [0, 1])
@pytest.mark.parametrize('lines,n', [(2048, 8192), (5000, 1000), (2048, 40000), (4096, 4)])
def test_builtin_entry_point_with_many_lines(lines, n, op):
    import torch
    lib = launcher.library()
    rs = np.random.RandomState(n)
    x = (rs.normal(0, 1, (lines, n)) if op == 0 else rs.uniform(0.999, 1.001, (lines, n))).astype(np.float32)
    d = torch.from_numpy(x).cuda()
    out = torch.empty_like(d)
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(lines, n))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    launcher.check(lib.ovl_scan_f32(op, d.data_ptr(), out.data_ptr(), lines, n, None, scratch.data_ptr(), nbytes, stream),
                   'scan')
    status = ctypes.c_int32(-1)
    launcher.check(lib.ovl_read_kernel_status(scratch.data_ptr(), stream, ctypes.byref(status)), 'status')
    assert status.value == 0
    x64 = x.astype(np.float64)
    want = (np.cumsum(x64, axis=1) if op == 0 else np.cumprod(x64, axis=1)).astype(np.float32)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1.3e-7, atol=0)


SHORT_SHAPES = [((65536, 32), 'float32'), ((16384, 128), 'float32'), ((70001, 16), 'float32'), ((4096, 16), 'float64'),
                ((32768, 8), 'int32'), ((65536, 4), 'float32'), ((16384, 64), 'uint8'), ((3, 9000, 64), 'float32'),
                ((8192, 32), 'float64'), ((4100, 256), 'float32'), ((2049, 512), 'float32'), ((1000, 256), 'float64'),
                ((1024, 512), 'int16'), ((70000, 100), 'float32'), ((40001, 36), 'float32'), ((9000, 500), 'float32'),
                ((5000, 250), 'float64'), ((20000, 12), 'int32'), ((2, 8200, 20), 'float32'), ((4099, 260), 'float32')]


@pytest.mark.parametrize('fn', ['cumsum', 'cumprod'])
@pytest.mark.parametrize('shape,dtype', SHORT_SHAPES)
def test_short_lines_are_streamed_flat(shape, dtype, fn):
    """Lines of at most 128 vectors (4 to 512 fp32 elements): as many whole lines as fit share a warp's chunk, a line
    may run from one row of the chunk into the next, the shuffle scans stop at line starts, memory is walked as one
    flat array."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    rs = np.random.RandomState(shape[-1] + len(shape))
    if dtype.startswith('float'):
        x = (rs.normal(0, 1, shape) if fn == 'cumsum' else rs.uniform(0.9, 1.1, shape)).astype(dtype)
    else:
        x = rs.randint(0 if dtype == 'uint8' else -2, 3, shape).astype(dtype)
    op = getattr(ns, fn)(x, axis=len(shape) - 1)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    plan = prog.plans[0]
    assert plan.meta['scan']['warp'] is not None and plan.meta['scan']['warp'].get('flat_vectors')
    if DRYRUN:
        return
    assert plan.last_variant == 'wscan'
    want = _reference(x, fn)
    if dtype == 'float32':
        np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)
    elif dtype == 'float64':
        np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-12)
    else:
        np.testing.assert_array_equal(got, want)


@pytest.mark.skipif(DRYRUN, reason='needs a device')
@pytest.mark.parametrize('op', [0, 1])
@pytest.mark.parametrize('lines,n', [(1 << 14, 4), (8192, 8), (5000, 16), (70001, 32), (1 << 14, 64), (1 << 17, 128),
                                     (1000, 64), (513, 128), (4097, 256), (300, 512), (1 << 15, 512), (40001, 100),
                                     (9000, 36), (3000, 500), (70000, 12), (1234, 260)])
def test_builtin_scan_of_short_lines(lines, n, op):
    """The built-in fp32 entry point on short lines (from 2^16 elements on: the flat kernel; below: the kernels for few
    lines), against the exact scan."""
    import torch
    lib = launcher.library()
    rs = np.random.RandomState(lines % 1000 + n)
    x = (rs.normal(0, 1, (lines, n)) if op == 0 else rs.uniform(0.9, 1.1, (lines, n))).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    out = torch.full_like(xd, float('nan'))
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(lines, n))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    launcher.check(lib.ovl_scan_f32(op, xd.data_ptr(), out.data_ptr(), lines, n, None, scratch.data_ptr(), nbytes, stream),
                   'scan')
    status = ctypes.c_int32(-1)
    launcher.check(lib.ovl_read_kernel_status(scratch.data_ptr(), stream, ctypes.byref(status)), 'status')
    assert status.value == 0
    wide = x.astype(np.float64)
    want = (np.cumsum(wide, axis=1) if op == 0 else np.cumprod(wide, axis=1)).astype(np.float32)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1.3e-7, atol=0)
