"""The multi-rank logic of the sharded scan on CPU: shard bounds, carry computation, and the exchange step run as
two gloo ranks (one process each).  The device kernels are covered by the GPU tests; here the collective and
the host arithmetic around it are."""
import os
import socket

import numpy as np
import pytest

from opveclib_b200 import parallel


def test_shard_bounds_cover_the_axis():
    for length in (1, 7, 8, 1000, 2 ** 31):
        for world in (1, 2, 3, 4, 8):
            edges = [parallel.shard_bounds(length, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == length
            for (a, b), (c, d) in zip(edges, edges[1:]):
                assert b == c and b >= a and d >= c
            sizes = [b - a for a, b in edges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_bounds(10, 4, 4)
    x = np.arange(10)
    assert np.array_equal(np.concatenate([parallel.shard_leading_axis(x, r, 3) for r in range(3)]), x)


@pytest.mark.parametrize('op', ['add', 'mul'])
@pytest.mark.parametrize('world', [1, 2, 4, 8])
def test_host_statement_of_the_three_steps(op, world):
    rs = np.random.RandomState(world)
    x = (rs.normal(0, 1, 10007) if op == 'add' else rs.uniform(0.99, 1.01, 10007)).astype(np.float32)
    shards = [parallel.shard_leading_axis(x, r, world) for r in range(world)]
    got = np.concatenate(parallel.sharded_scan_host(shards, op))
    x64 = x.astype(np.float64)
    want = (np.cumsum(x64) if op == 'add' else np.cumprod(x64)).astype(np.float32)
    # fp64 carry + fp64 running value: the sharded result is the correctly rounded exact scan up to one ulp
    np.testing.assert_allclose(got, want, rtol=2e-7, atol=0)


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_rank(rank, world, port, op, queue):
    import torch
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        rs = np.random.RandomState(5)
        x = (rs.normal(0, 1, 4099) if op == 'add' else rs.uniform(0.99, 1.01, 4099)).astype(np.float32)
        mine = parallel.shard_leading_axis(x, rank, world)
        m64 = mine.astype(np.float64)
        total = torch.tensor([m64.sum() if op == 'add' else m64.prod()], dtype=torch.float64)
        totals = torch.zeros(world, dtype=torch.float64)
        dist.all_gather_into_tensor(totals, total)
        carry = parallel.exclusive_carry(totals.numpy(), rank, op)
        run = np.cumsum(m64) + carry if op == 'add' else np.cumprod(m64) * carry
        queue.put((rank, run.astype(np.float32)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('op', ['add', 'mul'])
def test_carry_exchange_with_two_gloo_ranks(op):
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    world, port = 2, _free_port()
    procs = [ctx.Process(target=_gloo_rank, args=(r, world, port, op, queue)) for r in range(world)]
    for p in procs:
        p.start()
    parts = dict(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    rs = np.random.RandomState(5)
    x = (rs.normal(0, 1, 4099) if op == 'add' else rs.uniform(0.99, 1.01, 4099)).astype(np.float32)
    x64 = x.astype(np.float64)
    want = (np.cumsum(x64) if op == 'add' else np.cumprod(x64)).astype(np.float32)
    got = np.concatenate([parts[r] for r in range(world)])
    np.testing.assert_allclose(got, want, rtol=2e-7, atol=0)


def _gloo_reduce_rank(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        rs = np.random.RandomState(9)
        a, b = rs.normal(0, 1, 5001), rs.normal(0, 1, 5001)
        mine_a, mine_b = (parallel.shard_leading_axis(v, rank, world) for v in (a, b))
        red = parallel.ShardedReduce('add', device='cpu')
        # a dot product over a sharded vector: the rank's partial, then the exchange
        dot = red.combine(torch.tensor([np.dot(mine_a, mine_b)], dtype=torch.float64))
        # column sums over sharded rows, and a product
        m = rs.uniform(0.9, 1.1, (40, 6))
        cols = red.combine(torch.tensor(parallel.shard_leading_axis(m, rank, world).sum(axis=0)))
        prod = parallel.ShardedReduce('mul', device='cpu').combine(
            torch.tensor(parallel.shard_leading_axis(m, rank, world).prod(axis=0)))
        queue.put((rank, dot.numpy(), cols.numpy(), prod.numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_partial_exchange_of_a_sharded_reduction_with_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    world, port = 2, _free_port()
    procs = [ctx.Process(target=_gloo_reduce_rank, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, rest) for r, *rest in (queue.get(timeout=120) for _ in range(world)))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    rs = np.random.RandomState(9)
    a, b = rs.normal(0, 1, 5001), rs.normal(0, 1, 5001)
    m = rs.uniform(0.9, 1.1, (40, 6))
    for r in range(world):
        dot, cols, prod = got[r]
        np.testing.assert_allclose(dot, [np.dot(a, b)], rtol=1e-12)
        np.testing.assert_allclose(cols, m.sum(axis=0), rtol=1e-13)
        np.testing.assert_allclose(prod, m.prod(axis=0), rtol=1e-12)
    # every rank holds the same bits
    for x, y in zip(got[0], got[1]):
        assert np.array_equal(x, y)


def test_combine_partials_is_rank_ordered():
    parts = np.array([[1e16, 1.0], [1.0, 2.0], [-1e16, 3.0]])
    assert parallel.combine_partials(parts, 'add').tolist() == [(1e16 + 1.0) - 1e16, 6.0]
    assert parallel.combine_partials(parts[:, 1:], 'mul').tolist() == [6.0]
    with pytest.raises(ValueError):
        parallel.combine_partials(parts, 'max')


def _gloo_halo_rank(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        x = np.arange(11, dtype=np.float32)
        mine = torch.from_numpy(np.ascontiguousarray(parallel.shard_leading_axis(x, rank, world)))
        first = parallel.ShardedShift().halo(mine[-1:])
        queue.put((rank, first.numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_halo_of_a_sharded_cyclic_shift_with_two_gloo_ranks():
    """Every rank receives the last element of the rank before it (rank 0: of the last rank)."""
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    world, port = 2, _free_port()
    procs = [ctx.Process(target=_gloo_halo_rank, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # shards of arange(11): [0..5] and [6..10]
    assert got[0].tolist() == [10.0] and got[1].tolist() == [5.0]
