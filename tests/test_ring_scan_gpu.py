"""The single-launch scan of one long line (ring scan): built-in fp32 entry point and generated kernels.

Checked against the exact scan computed in fp64 (or integer arithmetic) on the host, at sizes that exercise one
wave, several waves, partial last waves, ragged last tiles and the carry; and against the three streaming passes
(`ovl_scan_f32_begin` / `_finish`), which must give the same values."""
import ctypes

import numpy as np
import pytest

import cases
from helpers import DRYRUN
from opveclib_b200 import launcher

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(DRYRUN, reason='needs a device')]

TILE = 8192


def _sm_count():
    import torch
    return torch.cuda.get_device_properties(0).multi_processor_count


def _scan(x, op, carry=None):
    import torch
    lib = launcher.library()
    stream = torch.cuda.current_stream().cuda_stream
    n = x.numel()
    out = torch.empty_like(x)
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(1, n))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
    c = None if carry is None else torch.tensor([carry], dtype=torch.float64, device='cuda')
    launcher.check(lib.ovl_scan_f32(op, x.data_ptr(), out.data_ptr(), 1, n, None if c is None else c.data_ptr(),
                                    scratch.data_ptr(), nbytes, stream), 'scan')
    status = ctypes.c_int32(-1)
    launcher.check(lib.ovl_read_kernel_status(scratch.data_ptr(), stream, ctypes.byref(status)), 'status')
    assert status.value == 0
    return out


def _exact(x, op, carry=None):
    x64 = x.astype(np.float64)
    ref = np.cumsum(x64) if op == 0 else np.cumprod(x64)
    if carry is not None:
        ref = ref + carry if op == 0 else ref * carry
    return ref.astype(np.float32)


def _sizes():
    g = 148
    return [TILE + 1, 2 * TILE, 20000, g * TILE, g * TILE + 1, (g + 1) * TILE - 3, 7 * g * TILE + 4097,
            13 * g * TILE + 5 * TILE + 2, 1 << 24]


@pytest.mark.parametrize('op', [0, 1])
@pytest.mark.parametrize('n', _sizes())
def test_long_line_is_the_rounded_exact_scan(op, n):
    import torch
    rs = np.random.RandomState(n % 977)
    x = (rs.normal(0, 1, n) if op == 0 else rs.uniform(0.9999, 1.0001, n)).astype(np.float32)
    carry = None if n % 2 else (3.25 if op == 0 else 1.5)
    got = _scan(torch.from_numpy(x).cuda(), op, carry).cpu().numpy()
    # fp64 accumulation: the correctly rounded exact prefix up to fp64 rounding of the reference itself
    np.testing.assert_allclose(got, _exact(x, op, carry), rtol=1.3e-7, atol=0)


def test_every_block_count_up_to_the_device(monkeypatch):
    """Lines of 2 .. SMs + 2 tiles: grids smaller than the device, exactly the device, and a second wave."""
    import torch
    sms = _sm_count()
    rs = np.random.RandomState(5)
    for tiles in [2, 3, 5, 31, 32, 33, sms - 1, sms, sms + 1, sms + 2]:
        n = tiles * TILE - 7
        x = rs.normal(0, 1, n).astype(np.float32)
        got = _scan(torch.from_numpy(x).cuda(), 0).cpu().numpy()
        np.testing.assert_allclose(got, _exact(x, 0), rtol=1.3e-7, atol=0)


def test_same_values_as_the_three_pass_scan():
    import torch
    lib = launcher.library()
    stream = torch.cuda.current_stream().cuda_stream
    n = 9 * 148 * TILE + 1234
    x = torch.from_numpy(np.random.RandomState(9).normal(0, 1, n).astype(np.float32)).cuda()
    ring = _scan(x, 0, 0.5)
    out = torch.empty_like(x)
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(1, n))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
    total = torch.zeros(1, dtype=torch.float64, device='cuda')
    carry = torch.tensor([0.5], dtype=torch.float64, device='cuda')
    launcher.check(lib.ovl_scan_f32_begin(0, x.data_ptr(), n, total.data_ptr(), scratch.data_ptr(), nbytes, stream), 'begin')
    launcher.check(lib.ovl_scan_f32_finish(0, x.data_ptr(), out.data_ptr(), n, carry.data_ptr(), scratch.data_ptr(), nbytes,
                                           stream), 'finish')
    torch.cuda.synchronize()
    a, b = ring.cpu().numpy(), out.cpu().numpy()
    # both are fp64 accumulations rounded once; the order of the fp64 additions differs, which may move a value
    # that sits on a rounding boundary by one unit in the last place
    np.testing.assert_allclose(a, b, rtol=1.3e-7, atol=0)
    assert (a != b).mean() < 1e-5
    assert abs(float(total.item()) - float(x.double().sum().item())) <= 1e-9 * n


def test_unaligned_pointers_take_the_streaming_passes():
    import torch
    n = 3 * 148 * TILE + 5
    x = np.random.RandomState(3).normal(0, 1, n + 1).astype(np.float32)
    dx = torch.from_numpy(x).cuda()[1:]            # 4-byte aligned only
    assert dx.data_ptr() % 16 != 0
    got = _scan(dx, 0).cpu().numpy()
    np.testing.assert_allclose(got, _exact(x[1:], 0), rtol=1.3e-7, atol=0)


@pytest.mark.parametrize('dtype', ['float32', 'float64', 'int32', 'uint8'])
@pytest.mark.parametrize('fn', ['cumsum', 'cumprod'])
def test_generated_scan_of_a_long_line(dtype, fn):
    """`accumulate` over a rank-1 tensor through the public API: the generated kernel is the ring scan."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    n = 5 * 148 * 2048 + 1003 if dtype == 'uint8' else 300007
    rs = np.random.RandomState(17)
    if dtype.startswith('float'):
        x = (rs.normal(0, 1, n) if fn == 'cumsum' else rs.uniform(0.9999, 1.0001, n)).astype(dtype)
    else:
        x = rs.randint(0, 3, n).astype(dtype)
    op = getattr(ns, fn)(x, axis=0)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    plan = prog.plans[0]
    assert plan.meta['scan']['ring'] is not None and plan.last_variant == 'ring'
    assert any(sym.endswith('_ring') for sym, _ in plan._variants)
    if dtype == 'float32':
        x64 = x.astype(np.float64)
        want = (np.cumsum(x64) if fn == 'cumsum' else np.cumprod(x64)).astype(np.float32)
        np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)
    elif dtype == 'float64':
        want = np.cumsum(x) if fn == 'cumsum' else np.cumprod(x)
        np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-9)
    else:
        # integer scans wrap exactly like the serial loop of the reference's operator
        want = (np.cumsum(x, dtype=x.dtype) if fn == 'cumsum' else np.cumprod(x, dtype=x.dtype))
        np.testing.assert_array_equal(got, want)


def test_a_wait_that_nothing_satisfies_ends_with_a_status_not_a_hang():
    """The library's self-test entry point withholds one block's aggregates: every block's bounded wait expires
    (the self-test's bound is 2^27 clock cycles, about 70 ms, so that the device is not held for long), the kernel
    returns, the status word says OVL_ERR_TIMEOUT - and the same context then scans the same data correctly."""
    import time
    import torch
    lib = launcher.library()
    stream = torch.cuda.current_stream().cuda_stream
    n = 6 * TILE
    x = np.random.RandomState(8).normal(0, 1, n).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    out = torch.empty_like(dx)
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(1, n))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
    t0 = time.time()
    launcher.check(lib.ovl_selftest_scan_timeout(dx.data_ptr(), out.data_ptr(), n, scratch.data_ptr(), nbytes, stream),
                   'self-test launch')
    status = ctypes.c_int32(-1)
    launcher.check(lib.ovl_read_kernel_status(scratch.data_ptr(), stream, ctypes.byref(status)), 'status')
    elapsed = time.time() - t0
    assert status.value == 8                      # OVL_ERR_TIMEOUT
    assert 0.02 < elapsed < 10.0
    assert lib.ovl_status_string(status.value).decode().startswith('bounded device-side wait')
    got = _scan(dx, 0).cpu().numpy()
    np.testing.assert_allclose(got, _exact(x, 0), rtol=1.3e-7, atol=0)


def _scan_lines(x2d, op):
    import torch
    lib = launcher.library()
    stream = torch.cuda.current_stream().cuda_stream
    lines, n = x2d.shape
    out = torch.empty_like(x2d)
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(lines, n))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
    launcher.check(lib.ovl_scan_f32(op, x2d.data_ptr(), out.data_ptr(), lines, n, None, scratch.data_ptr(), nbytes, stream),
                   'scan')
    status = ctypes.c_int32(-1)
    launcher.check(lib.ovl_read_kernel_status(scratch.data_ptr(), stream, ctypes.byref(status)), 'status')
    assert status.value == 0
    return out


@pytest.mark.parametrize('op', [0, 1])
@pytest.mark.parametrize('lines,n', [(2, 2 * TILE), (3, 2 * TILE + 4), (7, 5 * TILE - 8), (40, 9 * TILE + 12),
                                     (300, TILE + 4), (5, 148 * TILE + 2 * TILE), (2, 3 * 148 * TILE + 100)])
def test_several_long_lines_in_one_launch(lines, n, op):
    """Lines of several tiles each: tiles are numbered line by line, waves cross line boundaries, prefixes restart
    at every line start (line lengths divisible by four, so every line starts on a 16-byte boundary)."""
    import torch
    rs = np.random.RandomState(lines * 31 + n % 97)
    x = (rs.normal(0, 1, (lines, n)) if op == 0 else rs.uniform(0.9999, 1.0001, (lines, n))).astype(np.float32)
    got = _scan_lines(torch.from_numpy(x).cuda(), op).cpu().numpy()
    x64 = x.astype(np.float64)
    want = (np.cumsum(x64, axis=1) if op == 0 else np.cumprod(x64, axis=1)).astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)


@pytest.mark.parametrize('layout', ['grouped', 'waves'])
@pytest.mark.parametrize('op', [0, 1])
@pytest.mark.parametrize('lines,n', [(16, 20 * TILE + 8), (64, 6 * TILE + 16), (145, TILE + 4), (148, 4 * TILE),
                                     (296, 2 * TILE + 8), (1000, 3 * TILE + 4), (2000, 2 * TILE - 4)])
def test_lines_scanned_by_groups_of_blocks(lines, n, op, layout, monkeypatch):
    """Line counts for which every line gets a group of blocks of its own when that keeps the grid busy (16 lines: nine
    blocks each; from 148 lines on a block walks down its lines alone; 64 lines would leave a seventh of the grid
    idle and stay with waves), and the same shapes with waves that cross line ends forced."""
    import torch
    if layout == 'waves':
        monkeypatch.setenv('OVL_RING_LAYOUT', 'waves')
    rs = np.random.RandomState(lines + n % 89)
    x = (rs.normal(0, 1, (lines, n)) if op == 0 else np.exp(rs.uniform(-1e-3, 1e-3, (lines, n)))).astype(np.float32)
    got = _scan_lines(torch.from_numpy(x).cuda(), op).cpu().numpy()
    x64 = x.astype(np.float64)
    want = (np.cumsum(x64, axis=1) if op == 0 else np.cumprod(x64, axis=1)).astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)


@pytest.mark.parametrize('shape,dtype', [((4, 4, 70000), np.float32), ((20, 50000), np.float64), ((148, 20000), np.int32)])
def test_generated_scan_with_a_group_of_blocks_per_line(shape, dtype):
    from opveclib_b200 import runtime
    ns = cases.impl()
    rs = np.random.RandomState(29)
    x = (rs.randint(-9, 9, shape) if dtype == np.int32 else rs.normal(0, 1, shape)).astype(dtype)
    op = ns.cumsum(x, axis=len(shape) - 1)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    plan = prog.plans[0]
    assert plan.meta['scan']['ring']['layout'] == 'grouped' and plan.last_variant == 'ring'
    if dtype == np.int32:
        assert np.array_equal(got, np.cumsum(x, axis=-1, dtype=np.int32))
    else:
        want = np.cumsum(x.astype(np.float64), axis=-1)
        if dtype == np.float32:
            np.testing.assert_allclose(got, want.astype(np.float32), rtol=1.3e-7, atol=0)
        else:       # both sides add in fp64, in different orders
            bound = 1e-12 * (np.abs(want) + np.abs(want).max(axis=-1, keepdims=True))
            assert np.all(np.abs(got - want) <= bound)


def test_generated_scan_of_several_long_lines_along_the_last_axis():
    from opveclib_b200 import runtime
    ns = cases.impl()
    x = np.random.RandomState(23).normal(0, 1, (3, 5, 40000)).astype(np.float32)
    op = ns.cumsum(x, axis=2)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    plan = prog.plans[0]
    assert plan.meta['scan']['ring'] is not None and plan.last_variant == 'ring'
    want = np.cumsum(x.astype(np.float64), axis=2).astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)


@pytest.mark.parametrize('lines,n', [(32768, 64), (40001, 100), (70000, 512)])
def test_tens_of_thousands_of_short_lines(lines, n):
    """From 32768 lines on the warp-per-line kernel is launched with one line per warp in blocks of four warps (the
    hardware hands out blocks as earlier ones finish) instead of resident warps that walk the lines: through the
    C entry point and through a generated cumsum."""
    import torch
    from opveclib_b200 import runtime
    rs = np.random.RandomState(lines % 1000 + n)
    x = rs.normal(0, 1, (lines, n)).astype(np.float32)
    want = np.cumsum(x.astype(np.float64), axis=1).astype(np.float32)
    got = _scan_lines(torch.from_numpy(x).cuda(), 0).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)
    ns = cases.impl()
    op = ns.cumsum(x, axis=1)
    got = ns.ovl.evaluate([op])
    prog, _ = runtime.compile_outputs([op])
    assert prog.plans[0].last_variant == 'wscan'
    assert runtime.warp_scan_shape(lines, 148) == ((lines + 3) // 4, 128)
    np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)
