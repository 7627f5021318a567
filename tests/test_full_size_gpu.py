"""Parity at the full sizes of the benchmark configurations.

Where the CPU oracle finishes in seconds (configs 1 and 3) the whole result is compared with it.  For the
configurations that are too large for that, properties that do not depend on the size are checked on the full
tensors, and the oracle is run on samples:

* element-wise graphs are point-wise, so the oracle evaluated on a random sample of input elements must agree
  with the same elements of the full-size result; and evaluating row slabs separately must give bit-identical
  rows (how the multi-GPU run shards config 4);
* scans: first differences of the result reproduce the input, the last element of a line is the fp64 total of
  the line, results agree with a chunked fp64 scan carried on the device, sampled lines agree with the oracle,
  and shards scanned with carries reproduce the unsharded result exactly.
"""
import numpy as np
import pytest

import cases
from helpers import DRYRUN, assert_close, assert_exact

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(DRYRUN, reason='needs a device')]


def test_config1_full_size_against_the_oracle():
    from oracle import runner
    ns = cases.impl()
    x = np.random.RandomState(1).uniform(-1, 1, 1 << 20).astype(np.float32)
    chain, shift = cases.c1_chain(ns, x), cases.user_ops(ns).shift_cyclic(x)
    got_chain, got_shift = ns.ovl.evaluate([chain, shift])
    want_chain, want_shift = runner.evaluate([chain, shift])
    assert_exact(got_shift, want_shift, 'shift_cyclic 2^20')                       # index work: bit-exact
    assert_exact(got_shift, np.roll(x, 1), 'shift_cyclic 2^20 vs roll')
    assert_close(got_chain, want_chain, rtol=1e-5, atol=1e-6, what='c1 chain 2^20')
    inside = np.abs(got_chain.astype(np.float64) - want_chain) <= 1e-5 * np.abs(want_chain)
    assert inside.mean() > 0.999


def test_config3_full_size_against_the_oracle():
    from oracle import runner
    ns = cases.impl()
    rs = np.random.RandomState(3)
    g = rs.normal(0, 1, (512, 4096)).astype(np.float32)
    c = rs.normal(0, 1, (512, 1024)).astype(np.float32)
    dc = rs.normal(0, 0.1, (512, 1024)).astype(np.float32)
    dh = rs.normal(0, 0.1, (512, 1024)).astype(np.float32)
    fwd = ns.lstm(g, c, forget_bias=0.0)
    bwd = ns.lstm_grad(g, c, dc, dh, forget_bias=0.0)
    outs = [fwd[0], fwd[1], bwd[0], bwd[1]]
    got = ns.ovl.evaluate(outs)
    want = runner.evaluate(outs)
    for name, a, b in zip(('new_c', 'new_h', 'd_concat', 'd_c'), got, want):
        scale = float(np.abs(b).max())
        assert_close(a, b, rtol=1e-5, atol=1e-6 * scale, what='lstm ' + name)
        inside = np.abs(a.astype(np.float64) - b) <= 1e-5 * np.abs(b)
        assert inside.mean() > 0.995, name


def test_config4_full_size_samples_and_slab_invariance():
    import torch
    from oracle import runner
    ns = cases.impl()
    rows, cols = 8, 1 << 27
    gen = torch.Generator(device='cuda')
    gen.manual_seed(4)
    x = torch.empty((rows, cols), dtype=torch.float32, device='cuda').uniform_(-2, 2, generator=gen)
    y = ns.ovl.evaluate(cases.chain16(ns, x))
    assert y.shape == x.shape and bool(torch.isfinite(y).all())
    # point-wise: the oracle on 2^20 sampled elements (plus the corners) against the same elements of y
    idx = torch.randint(0, rows * cols, (1 << 20,), device='cuda', generator=gen)
    idx[:4] = torch.tensor([0, cols - 1, rows * cols - cols, rows * cols - 1], device='cuda')
    xs = x.reshape(-1)[idx].cpu().numpy()
    want = runner.evaluate(cases.chain16(ns, xs))
    got = y.reshape(-1)[idx].cpu().numpy()
    assert_close(got, want, rtol=1e-5, atol=1e-6 * float(np.abs(want).max()), what='chain16 samples')
    inside = np.abs(got.astype(np.float64) - want) <= 1e-5 * np.abs(want)
    assert inside.mean() > 0.995
    # sharding along axis 0: every slab evaluated on its own gives the same bits
    for parts in (2, 8):
        step = rows // parts
        for r in (0, parts - 1):
            slab = x[r * step:(r + 1) * step]
            ys = ns.ovl.evaluate(cases.chain16(ns, slab))
            assert torch.equal(ys, y[r * step:(r + 1) * step])


def test_config2_full_size_scans():
    import torch
    from oracle import runner
    ns = cases.impl()
    gen = torch.Generator(device='cuda')
    gen.manual_seed(2)
    for op, name in ((ns.cumsum, 'cumsum'), (ns.cumprod, 'cumprod')):
        x = torch.empty((4096, 8192), dtype=torch.float32, device='cuda')
        x = x.normal_(0, 1, generator=gen) if name == 'cumsum' else x.uniform_(0.99, 1.01, generator=gen)
        y = ns.ovl.evaluate(op(x, axis=1))
        x64 = x.double()
        exact = torch.cumsum(x64, 1) if name == 'cumsum' else torch.cumprod(x64, 1)
        # fp64 accumulation: the result is the exact scan rounded to fp32
        assert torch.equal(y, exact.float()) or \
            float(((y.double() - exact).abs() / exact.abs().clamp_min(1e-30)).max()) < 1.2e-7
        # sampled lines against the reference's serial fp32 loop (the oracle): it differs by its own rounding
        rows = [0, 1, 2047, 4095] + list(np.random.RandomState(5).randint(0, 4096, 28))
        xs = x[rows].cpu().numpy()
        want = runner.evaluate(op(xs, axis=1))
        got = y[rows].cpu().numpy()
        line_max = np.abs(want.astype(np.float64)).max(axis=1, keepdims=True)
        assert_close(got, want, rtol=1e-5, atol=1e-5 * line_max * np.ones(want.shape), what=name + ' sampled lines')


def test_config5_full_size_scan_properties_and_sharding():
    import ctypes
    import torch
    from opveclib_b200 import launcher, parallel
    n = 1 << 31
    gen = torch.Generator(device='cuda')
    gen.manual_seed(5)
    x = torch.empty(n, dtype=torch.float32, device='cuda').normal_(0, 1, generator=gen)
    scan = parallel.ShardedScan(n, 'add')
    y = scan(x)
    scan.check_status()
    # chunked fp64 scan with a carried total: the exact answer rounded to fp32
    carry = torch.zeros((), dtype=torch.float64, device='cuda')
    worst_loose, worst_tight = 0.0, 0.0
    chunk = 1 << 27
    for lo in range(0, n, chunk):
        ref = torch.cumsum(x[lo:lo + chunk].double(), 0) + carry
        carry = ref[-1].clone()
        err = (y[lo:lo + chunk].double() - ref).abs()
        # two fp64 summation orders differ by ~1e-10 absolute after 2^31 terms of this size; where the running sum
        # crosses zero that is no longer small relative to the value, hence the absolute floor of 1e-6
        worst_loose = max(worst_loose, float((err - 1e-5 * ref.abs()).max()))
        worst_tight = max(worst_tight, float((err - 6.0e-8 * ref.abs()).max()))
        del ref, err
    assert worst_loose <= 1e-6, worst_loose          # stated tolerance: rtol 1e-5 against the fp64 run
    assert worst_tight <= 1e-6, worst_tight          # in fact the fp64 result rounded once to fp32
    # first differences give the input back (to the rounding of the two neighbours)
    i = torch.randint(1, n, (1 << 22,), device='cuda', generator=gen)
    diff = y[i].double() - y[i - 1].double()
    tol = 1.2e-7 * (y[i].abs() + y[i - 1].abs()).double() + 1e-12
    assert bool(((diff - x[i].double()).abs() <= tol).all())
    # eight contiguous shards with carries reproduce the unsharded result bit for bit
    lib = launcher.library()
    stream = torch.cuda.current_stream().cuda_stream
    world = 8
    totals = torch.zeros(world, dtype=torch.float64, device='cuda')
    m = n // world
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(1, m))
    scratch = [torch.empty(nbytes, dtype=torch.uint8, device='cuda') for _ in range(world)]
    for r in range(world):
        launcher.check(lib.ovl_scan_f32_begin(0, x[r * m:].data_ptr(), m, totals[r:].data_ptr(), scratch[r].data_ptr(), nbytes,
                                              stream), 'begin')
    carries = torch.cumsum(totals, 0) - totals
    out = torch.empty(m, dtype=torch.float32, device='cuda')
    for r in (0, 3, 7):
        launcher.check(lib.ovl_scan_f32_finish(0, x[r * m:].data_ptr(), out.data_ptr(), m, carries[r:].data_ptr(),
                                               scratch[r].data_ptr(), nbytes, stream), 'finish')
        status = ctypes.c_int32(-1)
        lib.ovl_read_kernel_status(scratch[r].data_ptr(), stream, ctypes.byref(status))
        assert status.value == 0
        same = torch.equal(out, y[r * m:(r + 1) * m])
        if not same:
            # the carry is one fp64 sum, the unsharded prefix another: they may differ in the last fp64 bits and
            # flip a rounding in rare elements
            ref = y[r * m:(r + 1) * m].double()
            assert bool(((out.double() - ref).abs() <= 1.2e-7 * ref.abs() + 1e-6).all())


def test_host_resident_long_line_through_evaluate():
    """`ovl.evaluate(cumsum(numpy array))` of a long line streams chunks through the device
    (`parallel.HostScan`); the result is the exact scan, as from device-resident data."""
    import torch
    ns = cases.impl()
    n = (1 << 26) + (1 << 25) + 777            # one whole chunk and a ragged second one
    x = np.random.RandomState(6).normal(0, 1, n).astype(np.float32)
    got = ns.ovl.evaluate(ns.cumsum(x, axis=0))
    assert isinstance(got, np.ndarray) and got.shape == (n,)
    dev = ns.ovl.evaluate(ns.cumsum(torch.from_numpy(x).cuda(), axis=0)).cpu().numpy()
    # both are fp64 accumulations rounded once; chunking changes the order of a few fp64 additions, which can move a
    # value that sits on a rounding boundary by one unit in the last place
    np.testing.assert_allclose(got, dev, rtol=1.3e-7, atol=0)
    assert (got != dev).mean() < 1e-6
    # numpy's serial fp64 sum carries its own rounding (about 1e-12 here), enough to move a value next to a zero
    # crossing by one unit in the last place: two units allowed
    want = np.cumsum(x.astype(np.float64)).astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=2.5e-7, atol=0)
