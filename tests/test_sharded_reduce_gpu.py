"""Reductions whose reduced axis is split over ranks (`parallel.ShardedReduce`): per-shard totals by
`ovl_reduce_f32`, per-shard operator results, and the exchange of the partials - emulated rank by rank on one
GPU (the kernels of different ranks never wait for each other) and, with two devices, over NCCL."""
import os
import socket

import numpy as np
import pytest

import cases
from helpers import DRYRUN
from opveclib_b200 import parallel

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(DRYRUN, reason='needs a device')
@pytest.mark.parametrize('op', ['add', 'mul'])
@pytest.mark.parametrize('world', [1, 2, 4, 8])
def test_shard_totals_combined_in_rank_order(op, world):
    import torch
    rs = np.random.RandomState(world)
    n = 1000003
    x = (rs.normal(0, 1, n) if op == 'add' else rs.uniform(0.99999, 1.00001, n)).astype(np.float32)
    red = parallel.ShardedReduce(op)
    partials = []
    for r in range(world):
        mine = np.ascontiguousarray(parallel.shard_leading_axis(x, r, world))
        partials.append(red.total(torch.from_numpy(mine).cuda()).clone())       # (world size 1: the shard's own total)
    got = parallel.combine_partials(torch.stack(partials), op).cpu().numpy()
    x64 = x.astype(np.float64)
    want = x64.sum() if op == 'add' else x64.prod()
    np.testing.assert_allclose(got, [want], rtol=1e-11, atol=1e-9 if op == 'add' else 0)
    with pytest.raises(ValueError):
        red.total(torch.zeros(4, dtype=torch.float64, device='cuda'))


def test_dot_product_over_a_sharded_vector():
    """Each rank evaluates the operator on its shard (the `_red` kernel); the partials are combined."""
    import torch
    ns = cases.impl()
    dot = cases.user_ops(ns).dot
    rs = np.random.RandomState(4)
    n, world = 40000, 4
    a, b = rs.normal(0, 1, n), rs.normal(0, 1, n)
    partials = []
    for r in range(world):
        sa, sb = (np.ascontiguousarray(parallel.shard_leading_axis(v, r, world))[None, :] for v in (a, b))
        partials.append(torch.as_tensor(np.asarray(ns.ovl.evaluate([dot(sa, sb)]))).reshape(-1))
    got = parallel.combine_partials(torch.stack(partials), 'add').numpy()
    if DRYRUN:
        return
    np.testing.assert_allclose(got, [np.dot(a, b)], rtol=1e-11, atol=1e-11)


def _nccl_rank(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        rs = np.random.RandomState(11)
        x = rs.normal(0, 1, 2000001).astype(np.float32)
        m = rs.normal(0, 1, (1000, 16)).astype(np.float32)
        red = parallel.ShardedReduce('add')
        total = red.total(torch.from_numpy(np.ascontiguousarray(parallel.shard_leading_axis(x, rank, world))).cuda())
        cols = red.combine(torch.from_numpy(parallel.shard_leading_axis(m, rank, world).astype(np.float64).sum(axis=0)).cuda())
        queue.put((rank, total.cpu().numpy(), cols.cpu().numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpus_exchange_partials_over_nccl():
    if DRYRUN:
        pytest.skip('needs devices')
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
    world = 2
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, rest) for r, *rest in (queue.get(timeout=300) for _ in range(world)))
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    rs = np.random.RandomState(11)
    x = rs.normal(0, 1, 2000001).astype(np.float32)
    m = rs.normal(0, 1, (1000, 16)).astype(np.float32)
    for r in range(world):
        np.testing.assert_allclose(got[r][0], [x.astype(np.float64).sum()], rtol=1e-11, atol=1e-9)
        np.testing.assert_allclose(got[r][1], m.astype(np.float64).sum(axis=0), rtol=1e-12, atol=1e-12)
    assert np.array_equal(got[0][0], got[1][0]) and np.array_equal(got[0][1], got[1][1])
