"""The cyclic shift of the documentation's first example on a vector that is split over ranks: the local shift by the
generated kernel plus one halo element from the rank before."""
import os
import socket

import numpy as np
import pytest

from helpers import DRYRUN
from opveclib_b200 import parallel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('dtype', [np.float32, np.int64])
@pytest.mark.parametrize('world', [1, 3, 4])
def test_ranks_emulated_one_after_the_other(world, dtype):
    if DRYRUN:
        pytest.skip('needs a device')
    import torch
    x = (np.random.RandomState(world).normal(0, 100, 100003)).astype(dtype)
    shards = [np.ascontiguousarray(parallel.shard_leading_axis(x, r, world)) for r in range(world)]
    lasts = [torch.from_numpy(s[-1:]).cuda() for s in shards]
    parts = []
    for r in range(world):
        op = parallel.ShardedShift()
        op.world, op.rank = world, r
        op.halo = lambda last, r=r: lasts[(r - 1) % world]          # what the all-gather delivers
        parts.append(op(torch.from_numpy(shards[r]).cuda()).cpu().numpy())
    assert np.array_equal(np.concatenate(parts), np.roll(x, 1))


def _nccl_rank(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        x = np.random.RandomState(6).normal(0, 1, 1000001).astype(np.float32)
        mine = torch.from_numpy(np.ascontiguousarray(parallel.shard_leading_axis(x, rank, world))).cuda()
        out = parallel.ShardedShift()(mine)
        queue.put((rank, out.cpu().numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpus_exchange_the_halo_over_nccl():
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
    got = dict(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    x = np.random.RandomState(6).normal(0, 1, 1000001).astype(np.float32)
    assert np.array_equal(np.concatenate([got[0], got[1]]), np.roll(x, 1))
