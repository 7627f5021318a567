"""The allocation-free scan entry point against the regular one.

``ovl_scan_f32_static`` exists for hosts that must not allocate device memory themselves - a plugin inside an
engine whose memory pool owns the GPU, or a loop that cannot tolerate the synchronisation an allocation brings -
so it keeps its tile descriptors in an array compiled into the library instead of taking scratch from the
caller.  It runs the same kernel as ``ovl_scan_f32``; the two must therefore agree bit for bit.  Two calls are
made back to back on one stream, with different sizes and operators, because the second call sees whatever the
first one left in the shared array and has to clear it itself.
"""
import ctypes

import numpy as np
import pytest

from helpers import DRYRUN
from opveclib_b200 import launcher

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(DRYRUN, reason='needs a device')]

STATIC_BYTES = 1 << 20


def _scan_both(lib, torch, op, x):
    lines, n = x.shape
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty_like(x)
    bytes_needed = int(lib.ovl_scan_f32_scratch_bytes(lines, n))
    scratch = torch.empty(bytes_needed, dtype=torch.uint8, device=x.device)
    launcher.check(lib.ovl_scan_f32(op, x.data_ptr(), want.data_ptr(), lines, n, None, scratch.data_ptr(), bytes_needed,
                                    stream), 'ovl_scan_f32')
    got = torch.full_like(x, float('nan'))
    launcher.check(lib.ovl_scan_f32_static(op, x.data_ptr(), got.data_ptr(), lines, n, None, stream),
                   'ovl_scan_f32_static')
    status = ctypes.c_int32(-1)
    launcher.check(lib.ovl_scan_f32_static_status(stream, ctypes.byref(status)), 'ovl_scan_f32_static_status')
    assert status.value == 0
    return got.cpu().numpy(), want.cpu().numpy()


def test_static_scratch_scan_matches_regular_scan_on_two_calls_in_a_row():
    import torch
    lib = launcher.library()
    gen = torch.Generator(device='cuda')
    gen.manual_seed(77)
    # first call: many lines of three tiles each, sum; leaves 900 descriptors behind in the shared array
    a = torch.empty((300, 9000), dtype=torch.float32, device='cuda').normal_(0, 1, generator=gen)
    got, want = _scan_both(lib, torch, 0, a)
    assert np.array_equal(got, want)
    ref = np.cumsum(a.cpu().numpy().astype(np.float64), axis=1)
    assert np.all(np.abs(got - ref) <= 1e-6 * (np.abs(ref) + 1))
    # second call: one long line, product; reuses the descriptors the first call dirtied
    b = torch.empty((1, 1 << 22), dtype=torch.float32, device='cuda').uniform_(0.9999, 1.0001, generator=gen)
    got, want = _scan_both(lib, torch, 1, b)
    assert np.array_equal(got, want)
    ref = np.cumprod(b.cpu().numpy().astype(np.float64), axis=1)
    np.testing.assert_allclose(got, ref, rtol=1e-6)


def test_static_scratch_scan_rejects_what_does_not_fit():
    import torch
    lib = launcher.library()
    x = torch.zeros(16, dtype=torch.float32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    # more tile descriptors than the fixed array holds: refused before anything is enqueued
    too_many_lines = STATIC_BYTES
    assert lib.ovl_scan_f32_scratch_bytes(too_many_lines, 16) > STATIC_BYTES
    assert lib.ovl_scan_f32_static(0, x.data_ptr(), x.data_ptr(), too_many_lines, 16, None, stream) == 10
    assert lib.ovl_scan_f32_static(0, x.data_ptr(), x.data_ptr(), 1, 1 << 40, None, stream) == 10
    assert lib.ovl_scan_f32_static(0, None, x.data_ptr(), 1, 16, None, stream) == 4
    assert lib.ovl_scan_f32_static(2, x.data_ptr(), x.data_ptr(), 1, 16, None, stream) == 11
    torch.cuda.synchronize()
