"""The scan across shard boundaries on GPUs: built-in reduction and carry-seeded scan kernels, and the NCCL
exchange when two devices are present."""
import ctypes
import os
import socket

import numpy as np
import pytest

from helpers import DRYRUN
from opveclib_b200 import launcher, parallel

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(DRYRUN, reason='needs a device')]


def _reference(x, op):
    x64 = x.astype(np.float64)
    return (np.cumsum(x64) if op == 'add' else np.cumprod(x64)).astype(np.float32)


@pytest.mark.parametrize('op', ['add', 'mul'])
@pytest.mark.parametrize('n', [1, 5, 8191, 8192, 8193, 100003, 1 << 21])
def test_single_rank_scan_is_the_rounded_exact_scan(op, n):
    import torch
    rs = np.random.RandomState(n % 1000)
    x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.99, 1.01, n)).astype(np.float32)
    scan = parallel.ShardedScan(n, op)
    y = scan(torch.from_numpy(x).cuda())
    scan.check_status()
    got = y.cpu().numpy()
    want = _reference(x, op)
    # fp64 accumulation: every element is the correctly rounded exact prefix (the fp64 reference itself carries
    # rounding of the order of 1e-16 * n, far below one fp32 ulp here)
    np.testing.assert_allclose(got, want, rtol=1.3e-7, atol=0)


@pytest.mark.parametrize('op', ['add', 'mul'])
@pytest.mark.parametrize('world', [2, 4, 8])
def test_rank_emulation_on_one_gpu_reduce_carry_scan(op, world):
    """All ranks' three steps run one after the other on one device through the C-ABI entry points; the
    concatenated result equals the unsharded scan.  (Kernels of different ranks never wait for each other, so
    running them back to back on one GPU is the same computation.)"""
    import torch
    lib = launcher.library()
    code = 0 if op == 'add' else 1
    n = 50000 * world + 3
    rs = np.random.RandomState(world)
    x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.999, 1.001, n)).astype(np.float32)
    shards = [torch.from_numpy(np.ascontiguousarray(parallel.shard_leading_axis(x, r, world))).cuda()
              for r in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    totals = torch.zeros(world, dtype=torch.float64, device='cuda')
    for r, s in enumerate(shards):
        nbytes = int(lib.ovl_reduce_f32_scratch_bytes(s.numel()))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
        launcher.check(lib.ovl_reduce_f32(code, s.data_ptr(), s.numel(), totals[r:].data_ptr(), scratch.data_ptr(),
                                          nbytes, stream), 'reduce')
    host_totals = totals.cpu().numpy()
    for r, s in enumerate(shards):
        s64 = s.cpu().numpy().astype(np.float64)
        np.testing.assert_allclose(host_totals[r], s64.sum() if op == 'add' else s64.prod(), rtol=1e-12)
    parts = []
    for r, s in enumerate(shards):
        carry = torch.tensor([parallel.exclusive_carry(host_totals, r, op)], dtype=torch.float64, device='cuda')
        out = torch.empty_like(s)
        nbytes = int(lib.ovl_scan_f32_scratch_bytes(1, s.numel()))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
        launcher.check(lib.ovl_scan_f32(code, s.data_ptr(), out.data_ptr(), 1, s.numel(), carry.data_ptr(),
                                        scratch.data_ptr(), nbytes, stream), 'scan')
        status = ctypes.c_int32(-1)
        launcher.check(lib.ovl_read_kernel_status(scratch.data_ptr(), stream, ctypes.byref(status)), 'status')
        assert status.value == 0
        parts.append(out.cpu().numpy())
    np.testing.assert_allclose(np.concatenate(parts), _reference(x, op), rtol=1.3e-7, atol=0)


@pytest.mark.parametrize('op', ['add', 'mul'])
@pytest.mark.parametrize('world', [2, 8])
def test_rank_emulation_begin_exchange_finish(op, world):
    """The split entry points the sharded runner uses: begin (tile aggregates + shard total), host-side carry,
    finish (seeded scan), all ranks run one after the other on one device."""
    import torch
    lib = launcher.library()
    code = 0 if op == 'add' else 1
    n = 70001 * world + 5
    rs = np.random.RandomState(10 + world)
    x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.999, 1.001, n)).astype(np.float32)
    shards = [torch.from_numpy(np.ascontiguousarray(parallel.shard_leading_axis(x, r, world))).cuda()
              for r in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    totals = torch.zeros(world, dtype=torch.float64, device='cuda')
    scratches = []
    for r, s in enumerate(shards):
        nbytes = int(lib.ovl_scan_f32_scratch_bytes(1, s.numel()))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
        scratches.append((scratch, nbytes))
        launcher.check(lib.ovl_scan_f32_begin(code, s.data_ptr(), s.numel(), totals[r:].data_ptr(), scratch.data_ptr(),
                                              nbytes, stream), 'begin')
    host_totals = totals.cpu().numpy()
    parts = []
    for r, s in enumerate(shards):
        carry = torch.tensor([parallel.exclusive_carry(host_totals, r, op)], dtype=torch.float64, device='cuda')
        out = torch.empty_like(s)
        scratch, nbytes = scratches[r]
        launcher.check(lib.ovl_scan_f32_finish(code, s.data_ptr(), out.data_ptr(), s.numel(), carry.data_ptr(),
                                               scratch.data_ptr(), nbytes, stream), 'finish')
        parts.append(out.cpu().numpy())
    np.testing.assert_allclose(np.concatenate(parts), _reference(x, op), rtol=1.3e-7, atol=0)


@pytest.mark.parametrize('op', ['add', 'mul'])
@pytest.mark.parametrize('world', [2, 5, 8])
def test_rank_emulation_of_the_peer_exchange(op, world):
    """The pair whose totals travel through exchange buffers instead of a collective, with every rank's buffer on
    this one device: every rank's `begin` is enqueued before any rank's `finish`, so no kernel ever waits for a
    later launch.  Three epochs in a row reuse the buffers (two parities, tagged words, no reset)."""
    import torch
    lib = launcher.library()
    code = 0 if op == 'add' else 1
    shard = 8192 * 160 + 64          # (long enough for the scan's scratch to hold the reduction's partials too)
    n = shard * world
    stream = torch.cuda.current_stream().cuda_stream
    nwords = int(lib.ovl_peer_buffer_bytes()) // 8
    buffers = [torch.zeros(nwords, dtype=torch.int64, device='cuda') for _ in range(world)]
    exchanges = []
    for r in range(world):
        px = launcher.OvlPeerExchange()
        px.world, px.rank = world, r
        for q in range(world):
            px.buffers[q] = buffers[q].data_ptr()
        exchanges.append(px)
    nbytes = int(lib.ovl_scan_f32_scratch_bytes(1, shard))
    scratches = [torch.empty(nbytes, dtype=torch.uint8, device='cuda') for _ in range(world)]
    totals = torch.zeros(world, dtype=torch.float64, device='cuda')
    for epoch in (1, 2, 3):
        rs = np.random.RandomState(100 * world + epoch)
        x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.9999, 1.0001, n)).astype(np.float32)
        shards = [torch.from_numpy(x[r * shard:(r + 1) * shard]).cuda() for r in range(world)]
        outs = [torch.empty_like(s) for s in shards]
        for r in range(world):
            exchanges[r].epoch = epoch
            launcher.check(lib.ovl_scan_f32_begin_peer(code, shards[r].data_ptr(), shard, totals[r:].data_ptr(),
                                                       scratches[r].data_ptr(), nbytes, ctypes.byref(exchanges[r]),
                                                       stream), 'begin')
        for r in range(world):
            launcher.check(lib.ovl_scan_f32_finish_peer(code, shards[r].data_ptr(), outs[r].data_ptr(), shard,
                                                        scratches[r].data_ptr(), nbytes, ctypes.byref(exchanges[r]),
                                                        stream), 'finish')
        for r in range(world):
            status = ctypes.c_int32(-1)
            launcher.check(lib.ovl_read_kernel_status(scratches[r].data_ptr(), stream, ctypes.byref(status)), 'status')
            assert status.value == 0
        got = np.concatenate([o.cpu().numpy() for o in outs])
        np.testing.assert_allclose(got, _reference(x, op), rtol=1.3e-7, atol=0)
    # arguments the pair refuses: an unaligned shard, a short shard, epoch 0
    bad = launcher.OvlPeerExchange()
    bad.world, bad.rank, bad.epoch = world, 0, 0
    for q in range(world):
        bad.buffers[q] = buffers[q].data_ptr()
    assert lib.ovl_scan_f32_begin_peer(code, shards[0].data_ptr(), shard, totals.data_ptr(), scratches[0].data_ptr(),
                                       nbytes, ctypes.byref(bad), stream) == 11
    bad.epoch = 4
    assert lib.ovl_scan_f32_begin_peer(code, shards[0].data_ptr() + 4, shard - 1, totals.data_ptr(),
                                       scratches[0].data_ptr(), nbytes, ctypes.byref(bad), stream) == 9
    assert lib.ovl_scan_f32_begin_peer(code, shards[0].data_ptr(), 4096, totals.data_ptr(), scratches[0].data_ptr(),
                                       nbytes, ctypes.byref(bad), stream) == 9


def test_single_pass_lookback_mode_agrees_with_three_pass_mode():
    """OVL_SCAN_MODE=lookback selects the decoupled look-back kernel for lines of several tiles; it is read once
    per process, so the check runs in a child process.  Both modes accumulate in fp64 and must give the same
    correctly rounded results."""
    import subprocess
    import sys
    code = """
import numpy as np, torch, ctypes, sys
sys.path.insert(0, %r)
from opveclib_b200 import launcher
lib = launcher.library()
rs = np.random.RandomState(3)
for lines, n, op in ((1, 300007, 0), (5, 20000, 0), (3, 40001, 1), (1, 1 << 22, 0)):
    x = (rs.normal(0, 1, (lines, n)) if op == 0 else rs.uniform(0.9999, 1.0001, (lines, n))).astype(np.float32)
    d = torch.from_numpy(x).cuda(); y = torch.empty_like(d)
    nb = int(lib.ovl_scan_f32_scratch_bytes(lines, n)); scratch = torch.empty(nb, dtype=torch.uint8, device='cuda')
    st = torch.cuda.current_stream().cuda_stream
    launcher.check(lib.ovl_scan_f32(op, d.data_ptr(), y.data_ptr(), lines, n, None, scratch.data_ptr(), nb, st), 'scan')
    status = ctypes.c_int32(-1); lib.ovl_read_kernel_status(scratch.data_ptr(), st, ctypes.byref(status))
    assert status.value == 0, status.value
    x64 = x.astype(np.float64)
    want = (np.cumsum(x64, axis=1) if op == 0 else np.cumprod(x64, axis=1)).astype(np.float32)
    np.testing.assert_allclose(y.cpu().numpy(), want, rtol=1.3e-7, atol=0)
print('lookback ok')
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OVL_SCAN_MODE='lookback')
    res = subprocess.run([sys.executable, '-c', code], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and 'lookback ok' in res.stdout, res.stdout + res.stderr


def _nccl_rank(rank, world, port, op, n, queue, exchange='collective'):
    import torch
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        rs = np.random.RandomState(9)
        x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.999, 1.001, n)).astype(np.float32)
        mine = np.ascontiguousarray(parallel.shard_leading_axis(x, rank, world))
        scan = parallel.ShardedScan(mine.size, op, exchange=exchange)
        assert scan.exchange == exchange
        d = torch.from_numpy(mine).cuda()
        y = scan(d)
        for _ in range(3):              # the buffers of the exchange are reused call after call
            y = scan(d, out=y)
        scan.check_status()
        queue.put((rank, y.cpu().numpy()))
        dist.barrier()
        if scan.peer is not None:
            scan.peer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('op', ['add', 'mul'])
def test_two_gpus_exchange_totals_through_peer_memory(op):
    """Two processes, one GPU each: the reduction kernel stores the shard total into both ranks' exchange
    buffers, the scan kernel of each rank waits for both totals in its own buffer.  No collective between the two
    kernels."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    world, n = 2, 3000064
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, op, n, queue, 'peer')) for r in range(world)]
    for p in procs:
        p.start()
    parts = dict(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    rs = np.random.RandomState(9)
    x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.999, 1.001, n)).astype(np.float32)
    np.testing.assert_allclose(np.concatenate([parts[r] for r in range(world)]), _reference(x, op), rtol=1.3e-7,
                               atol=0)


@pytest.mark.parametrize('op', ['add', 'mul'])
def test_two_gpus_exchange_carries_over_nccl(op):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    world, n = 2, 300001
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, op, n, queue)) for r in range(world)]
    for p in procs:
        p.start()
    parts = dict(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    rs = np.random.RandomState(9)
    x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.999, 1.001, n)).astype(np.float32)
    np.testing.assert_allclose(np.concatenate([parts[r] for r in range(world)]), _reference(x, op), rtol=1.3e-7,
                               atol=0)


@pytest.mark.parametrize('op', ['add', 'mul'])
def test_host_resident_line_is_scanned_chunk_by_chunk(op):
    """`parallel.HostScan`: chunks of the line travel through the device while the previous one is scanned; the
    carry between chunks stays on the device in fp64, so the result is the exact scan of the whole line."""
    import torch
    n = 3 * (1 << 20) + 12345
    rs = np.random.RandomState(21)
    x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.99999, 1.00001, n)).astype(np.float32)
    host_in = torch.from_numpy(x).pin_memory()
    host_out = torch.empty(n, dtype=torch.float32).pin_memory()
    scan = parallel.HostScan(chunk_len=1 << 20, op=op)
    scan(host_in, host_out)
    np.testing.assert_allclose(host_out.numpy(), _reference(x, op), rtol=1.3e-7, atol=0)
    # a second call reuses the buffers
    scan(host_in, host_out)
    np.testing.assert_allclose(host_out.numpy(), _reference(x, op), rtol=1.3e-7, atol=0)
