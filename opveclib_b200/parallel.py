"""Single-box data parallelism: shard the leading axis over the ranks of a ``torch.distributed`` group.

Workers of an operator are independent by construction (documentation/programming.rst:21 of the reference), so
an element-wise or fused operator graph whose tensors all share the leading axis runs unchanged on each rank's
slab - no communication.  The one exchange this backend knows is the carry of a scan that runs *along* the
sharded axis (the reference has no multi-GPU support at all; its rank-1 ``accumulate`` is a single worker,
opveclib/examples/test_accumulate.py:40-41):

1. every rank reads its shard once and forms the shard total in fp64 (``ovl_scan_f32_begin``);
2. the totals are all-gathered (8 bytes per rank, NCCL on GPUs, gloo in CPU tests) into local memory;
3. every rank combines the totals of the ranks before it into its carry and scans its shard seeded with it
   (``ovl_scan_f32_finish``: the ring scan, one launch).

On GPUs that can map each other's memory the exchange needs no collective call: the kernel of step 1 stores its
total straight into every rank's exchange buffer (plain stores over NVLink), and the scan kernel of step 3 starts
by waiting - bounded - for the totals of the epoch in its own buffer and folds them itself
(``ovl_scan_f32_begin_peer`` / ``ovl_scan_f32_finish_peer``; ``exchange='peer'``).  Two kernels per step and
nothing in between.

Per element this moves 4 bytes in step 1 and 8 in step 3: a shard's total is only known after all of it has been
read, so every shard but the first is read twice - 12 bytes per element against the 8 of the one-GPU scan.

A reduction along the sharded axis exchanges partial results the same way (``ShardedReduce``): every rank reduces
its shard, the partials are all-gathered into local memory and combined in rank order on every rank.
"""
import ctypes

import numpy as np

from . import launcher


def shard_bounds(length, rank, world_size):
    """[begin, end) of ``rank``'s contiguous shard of an axis of ``length`` elements: the first
    ``length % world_size`` ranks get one extra element."""
    if not 0 <= rank < world_size:
        raise ValueError('rank out of range')
    base, extra = divmod(length, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_leading_axis(array, rank, world_size):
    """The rank's slab of ``array`` along axis 0 (a view)."""
    begin, end = shard_bounds(array.shape[0], rank, world_size)
    return array[begin:end]


def exclusive_carry(totals, rank, op):
    """Combine the shard totals of the ranks before ``rank`` left to right, in fp64."""
    carry = np.float64(0.0 if op == 'add' else 1.0)
    for r in range(rank):
        carry = carry + np.float64(totals[r]) if op == 'add' else carry * np.float64(totals[r])
    return carry


def _op_code(op):
    if op not in ('add', 'mul'):
        raise ValueError("op must be 'add' or 'mul'")
    return 0 if op == 'add' else 1


class ShardedScan(object):
    """Inclusive cumsum / cumprod of a rank-1 fp32 tensor split contiguously over the ranks of ``group``.

    ``exchange``: 'peer' - totals travel through peer memory inside the two kernels (needs one GPU per rank on one
    box and 16-byte aligned shards longer than 8192 elements); 'collective' - ``all_gather`` of the totals between
    the two kernels; 'auto' (default) - 'peer' when it can be set up, else 'collective'.

    Buffers (scratch, totals, exchange buffer) are allocated once per instance; ``__call__`` enqueues the steps on
    torch's current stream and returns the rank's part of the result."""

    def __init__(self, shard_len, op='add', group=None, device=None, exchange='auto'):
        import torch
        import torch.distributed as dist
        if exchange not in ('auto', 'peer', 'collective'):
            raise ValueError("exchange must be 'auto', 'peer' or 'collective'")
        self.torch, self.dist = torch, dist
        self.op = op
        self.code = _op_code(op)
        self.group = group
        self.shard_len = int(shard_len)
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.device = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
        lib = launcher.library()
        self.lib = lib
        self.scan_bytes = int(lib.ovl_scan_f32_scratch_bytes(1, self.shard_len))
        self.scan_scratch = torch.empty(self.scan_bytes, dtype=torch.uint8, device=self.device)
        self.total = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.totals = torch.zeros(self.world, dtype=torch.float64, device=self.device)
        self.carry = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.launches = 0
        self.peer = None
        self.exchange = 'collective'
        if self.world > 1 and exchange in ('auto', 'peer'):
            # all ranks must take the same path: agree on whether every shard qualifies and every mapping worked
            try:
                votes = [None] * self.world
                # (the pair shares the scan's scratch, which must also hold the reduction's per-chunk partials)
                fits = self.shard_len > 8192 and \
                    self.scan_bytes >= 16 + int(lib.ovl_reduce_f32_scratch_bytes(self.shard_len))
                dist.all_gather_object(votes, fits and self.world <= launcher.MAX_PEERS, group=group)
                if not all(votes):
                    raise ValueError('the peer exchange needs shards of more than 8192 elements on at most %d ranks'
                                     % launcher.MAX_PEERS)
                self.peer = PeerTotals(self.world, self.rank, group, self.device)
                self.exchange = 'peer'
            except Exception:
                if exchange == 'peer':
                    raise
                self.peer = None

    def __call__(self, x, out=None):
        torch = self.torch
        if x.dtype != torch.float32 or x.dim() != 1 or x.numel() != self.shard_len or not x.is_contiguous():
            raise ValueError('expected a contiguous rank-1 float32 tensor of %d elements' % self.shard_len)
        if out is None:
            out = torch.empty_like(x)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if self.world == 1:
            launcher.check(self.lib.ovl_scan_f32(self.code, x.data_ptr(), out.data_ptr(), 1, self.shard_len, None,
                                                 self.scan_scratch.data_ptr(), self.scan_bytes, stream), 'scan')
            self.launches += 1
            return out
        if self.peer is not None:
            if x.data_ptr() % 16 or out.data_ptr() % 16:
                raise ValueError("the peer exchange needs 16-byte aligned shards: construct with exchange='collective'")
            px = self.peer.next_epoch()
            launcher.check(self.lib.ovl_scan_f32_begin_peer(self.code, x.data_ptr(), self.shard_len, self.total.data_ptr(),
                                                            self.scan_scratch.data_ptr(), self.scan_bytes, px, stream),
                           'shard total')
            launcher.check(self.lib.ovl_scan_f32_finish_peer(self.code, x.data_ptr(), out.data_ptr(), self.shard_len,
                                                             self.scan_scratch.data_ptr(), self.scan_bytes, px, stream),
                           'shard scan')
            self.launches += 2
            return out
        # step 1: the shard total
        launcher.check(self.lib.ovl_scan_f32_begin(self.code, x.data_ptr(), self.shard_len, self.total.data_ptr(),
                                                   self.scan_scratch.data_ptr(), self.scan_bytes, stream), 'shard totals')
        # step 2: exchange, carry = combination of the totals of the ranks before this one
        self.dist.all_gather_into_tensor(self.totals, self.total, group=self.group)
        if self.rank == 0:
            self.carry.fill_(0.0 if self.op == 'add' else 1.0)
        elif self.op == 'add':
            torch.sum(self.totals[:self.rank], dim=0, keepdim=True, out=self.carry)
        else:
            torch.prod(self.totals[:self.rank], dim=0, keepdim=True, out=self.carry)
        # step 3: the scan of the shard, seeded with the carry
        launcher.check(self.lib.ovl_scan_f32_finish(self.code, x.data_ptr(), out.data_ptr(), self.shard_len,
                                                    self.carry.data_ptr(), self.scan_scratch.data_ptr(),
                                                    self.scan_bytes, stream), 'shard scan')
        self.launches += 2
        return out

    def check_status(self):
        """Raise if a bounded wait inside the scan kernel expired."""
        status = ctypes.c_int32(0)
        stream = self.torch.cuda.current_stream(self.device).cuda_stream
        launcher.check(self.lib.ovl_read_kernel_status(self.scan_scratch.data_ptr(), stream, ctypes.byref(status)),
                       'reading scan status')
        if status.value != 0:
            raise launcher.OvlError(status.value, 'sharded scan')


class PeerTotals(object):
    """The exchange buffers of a sharded scan whose totals travel through peer memory: one small device buffer per
    rank, mapped into every other rank's process through CUDA IPC handles exchanged once over ``group``."""

    def __init__(self, world, rank, group, device):
        import torch
        import torch.distributed as dist
        if world > launcher.MAX_PEERS:
            raise ValueError('at most %d ranks' % launcher.MAX_PEERS)
        self.lib = launcher.library()
        self.world, self.rank = world, rank
        self.epoch = 0
        self.own = ctypes.c_void_p()
        self.opened = []
        handle = ctypes.create_string_buffer(launcher.PEER_HANDLE_BYTES)
        with torch.cuda.device(device):
            launcher.check(self.lib.ovl_peer_alloc(ctypes.byref(self.own), handle), 'allocating the exchange buffer')
            handles = [None] * world
            dist.all_gather_object(handles, (rank, bytes(handle.raw)), group=group)
            self.px = launcher.OvlPeerExchange()
            self.px.world, self.px.rank = world, rank
            ok = True
            for r, h in handles:
                if r == rank:
                    self.px.buffers[r] = self.own.value
                    continue
                p = ctypes.c_void_p()
                if self.lib.ovl_peer_open(h, ctypes.byref(p)) != 0:
                    ok = False
                    continue
                self.opened.append(p)
                self.px.buffers[r] = p.value
            # every rank must come to the same decision
            votes = [None] * world
            dist.all_gather_object(votes, ok, group=group)
            if not all(votes):
                self.close()
                raise RuntimeError('peer memory of another rank could not be mapped')

    def next_epoch(self):
        self.epoch += 1
        self.px.epoch = self.epoch
        return ctypes.byref(self.px)

    def close(self):
        for p in self.opened:
            self.lib.ovl_peer_close(p)
        self.opened = []
        if self.own:
            self.lib.ovl_peer_free(self.own)
            self.own = ctypes.c_void_p()


def combine_partials(partials, op='add'):
    """Combine per-rank partial results (first axis = rank) in rank order.  Works on numpy arrays and torch tensors;
    every rank calls it on the same gathered data and therefore gets bit-identical results."""
    if op not in ('add', 'mul'):
        raise ValueError("op must be 'add' or 'mul'")
    acc = partials[0]
    for r in range(1, len(partials)):
        acc = acc + partials[r] if op == 'add' else acc * partials[r]
    return acc


class ShardedReduce(object):
    """A reduction whose reduced axis is split over the ranks of ``group``: every rank reduces its own shard, the
    partial results are all-gathered into local memory and combined in rank order (the "partial exchange"; the
    reference has no multi-GPU support).  Two forms:

    ``total(x)``        sum / product of all elements of a contiguous fp32 tensor shard in fp64
                        (``ovl_reduce_f32``: one streaming read, fixed combination order), then the exchange;
    ``combine(partial)`` the exchange alone, for a partial result of any shape that an operator graph produced
                        from the rank's shard (a dot product over a sharded vector, column sums over sharded rows).
    Both return the same tensor on every rank."""

    def __init__(self, op='add', group=None, device=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.op = op
        self.code = _op_code(op)
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.device = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
        self.lib = launcher.library() if self.device.type == 'cuda' else None
        self._scratch = None
        self.partial = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.launches = 0

    def combine(self, partial):
        """All-gather ``partial`` (same shape and dtype on every rank) and combine the copies in rank order."""
        if self.world == 1:
            return partial
        torch = self.torch
        flat = partial.contiguous().view(-1)
        gathered = torch.empty(self.world * flat.numel(), dtype=partial.dtype, device=partial.device)
        self.dist.all_gather_into_tensor(gathered, flat, group=self.group)
        return combine_partials(gathered.view((self.world,) + tuple(partial.shape)), self.op)

    def total(self, x):
        """fp64 sum / product over all ranks' shards of a contiguous float32 CUDA tensor; a [1] float64 tensor."""
        torch = self.torch
        if x.dtype != torch.float32 or not x.is_contiguous() or not x.is_cuda:
            raise ValueError('expected a contiguous float32 CUDA tensor')
        n = x.numel()
        need = int(self.lib.ovl_reduce_f32_scratch_bytes(n))
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        launcher.check(self.lib.ovl_reduce_f32(self.code, x.data_ptr(), n, self.partial.data_ptr(),
                                               self._scratch.data_ptr(), self._scratch.numel(), stream), 'shard total')
        self.launches += 1
        return self.combine(self.partial)


class ShardedShift(object):
    """The cyclic shift of the documentation's first example (README.rst:40-74: ``out[i] = x[(i - 1) mod N]``,
    ``[0, 1, 2, 3, 4] -> [4, 0, 1, 2, 3]``) for a vector split contiguously over the ranks of ``group``: a rank's first
    output element is the LAST input element of the rank before it (of the last rank, for rank 0), everything else is
    local.  One element per rank is all-gathered into local memory (the halo), the rank's shard is shifted by the
    generated kernel, and the halo element replaces the one value the local shift wrapped around.  The reference has
    no multi-GPU support; on one rank this is the plain operator."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0

    def halo(self, last):
        """``last``: this rank's last input element as a one-element tensor.  Returns the element that belongs in front
        of this rank's shard: the last element of the rank before it."""
        import torch
        if self.world == 1:
            return last
        gathered = torch.empty(self.world, dtype=last.dtype, device=last.device)
        self.dist.all_gather_into_tensor(gathered, last.contiguous().view(1), group=self.group)
        return gathered[(self.rank - 1) % self.world].view(1)

    def __call__(self, x):
        """``x``: this rank's shard, a contiguous one-dimensional CUDA tensor.  Returns the rank's shard of the shifted
        vector (a CUDA tensor)."""
        from .examples.workloads import namespace, user_ops
        from .runtime import evaluate
        if x.dim() != 1 or not x.is_cuda or not x.is_contiguous():
            raise ValueError('expected a contiguous one-dimensional CUDA tensor')
        first = self.halo(x[-1:])                               # (enqueued before the kernel: they overlap)
        out = evaluate([user_ops(namespace()).shift_cyclic(x)], target_language='b200')
        out[0:1].copy_(first)
        return out


class HostScan(object):
    """Inclusive cumsum / cumprod of a rank-1 fp32 array that lives in HOST memory, on one GPU.

    The line is cut into chunks that travel through the device one after the other: while chunk i is scanned,
    chunk i+1 is on its way in and chunk i-1 on its way out, so both directions of the host link are busy at
    once and the device holds only a few chunks.  A chunk is scanned with the carry of everything before it
    (``ovl_scan_f32`` with a device-side fp64 carry); the carry advances by the chunk's fp64 total
    (``ovl_reduce_f32``), all on the device, so the host never waits inside the loop.  Results are those of the
    one-piece scan: fp64 accumulation, rounded once.  Pinned host arrays make the copies asynchronous."""

    def __init__(self, chunk_len=1 << 26, op='add', device=None):
        import torch
        self.torch = torch
        self.op = op
        self.code = _op_code(op)
        self.chunk_len = int(chunk_len)
        self.device = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
        self.lib = launcher.library()
        self.scan_bytes = int(self.lib.ovl_scan_f32_scratch_bytes(1, self.chunk_len))
        self.red_bytes = int(self.lib.ovl_reduce_f32_scratch_bytes(self.chunk_len))
        dev = self.device
        self.d_in = [torch.empty(self.chunk_len, dtype=torch.float32, device=dev) for _ in range(2)]
        self.d_out = [torch.empty(self.chunk_len, dtype=torch.float32, device=dev) for _ in range(2)]
        self.scan_scratch = torch.empty(self.scan_bytes, dtype=torch.uint8, device=dev)
        self.red_scratch = torch.empty(self.red_bytes, dtype=torch.uint8, device=dev)
        self.total = torch.zeros(1, dtype=torch.float64, device=dev)
        # the scan's status word (first four bytes of its scratch) and the worst status seen over the chunks
        self.status_word = self.scan_scratch[:4].view(torch.int32)
        self.status_seen = torch.zeros(1, dtype=torch.int32, device=dev)
        self.carries = None
        self.launches = 0

    def __call__(self, host_in, host_out):
        """``host_in`` / ``host_out``: rank-1 float32 torch CPU tensors of equal length (pinned for speed)."""
        torch = self.torch
        n = host_in.numel()
        if host_in.dtype != torch.float32 or host_out.dtype != torch.float32 or host_in.dim() != 1 or \
                host_out.numel() != n or not host_in.is_contiguous() or not host_out.is_contiguous():
            raise ValueError('expected contiguous rank-1 float32 host tensors of equal length')
        chunks = (n + self.chunk_len - 1) // self.chunk_len
        identity = 0.0 if self.op == 'add' else 1.0
        with torch.cuda.device(self.device):
            main = torch.cuda.current_stream()
            s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
            for st in (s_in, s_run, s_out):
                st.wait_stream(main)
            # carry in front of every chunk, advanced on the device
            with torch.cuda.stream(s_run):
                self.status_seen.zero_()
                carries = torch.full((chunks + 1,), identity, dtype=torch.float64, device=self.device)
            loaded, computed, stored = [None, None], [None, None], [None, None]
            for i in range(chunks):
                b = i % 2
                lo = i * self.chunk_len
                m = min(self.chunk_len, n - lo)
                with torch.cuda.stream(s_in):
                    if computed[b] is not None:
                        s_in.wait_event(computed[b])
                    self.d_in[b][:m].copy_(host_in[lo:lo + m], non_blocking=True)
                    loaded[b] = torch.cuda.Event()
                    loaded[b].record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(loaded[b])
                    if stored[b] is not None:
                        s_run.wait_event(stored[b])
                    sp = s_run.cuda_stream
                    launcher.check(self.lib.ovl_reduce_f32(self.code, self.d_in[b].data_ptr(), m, self.total.data_ptr(),
                                                           self.red_scratch.data_ptr(), self.red_bytes, sp), 'chunk total')
                    if self.op == 'add':
                        torch.add(carries[i:i + 1], self.total, out=carries[i + 1:i + 2])
                    else:
                        torch.mul(carries[i:i + 1], self.total, out=carries[i + 1:i + 2])
                    launcher.check(self.lib.ovl_scan_f32(self.code, self.d_in[b].data_ptr(), self.d_out[b].data_ptr(), 1, m,
                                                         carries[i:].data_ptr(), self.scan_scratch.data_ptr(),
                                                         self.scan_bytes, sp), 'chunk scan')
                    torch.maximum(self.status_seen, self.status_word, out=self.status_seen)
                    self.launches += 2
                    computed[b] = torch.cuda.Event()
                    computed[b].record(s_run)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(computed[b])
                    host_out[lo:lo + m].copy_(self.d_out[b][:m], non_blocking=True)
                    stored[b] = torch.cuda.Event()
                    stored[b].record(s_out)
            for st in (s_in, s_run, s_out):
                main.wait_stream(st)
            main.synchronize()
            self.carries = carries
            status = int(self.status_seen.item())
            self.status_seen.zero_()
            if status != 0:
                raise launcher.OvlError(status, 'host scan')
        return host_out


def sharded_scan_host(shards, op='add'):
    """Host-side statement of the three steps over a list of numpy shards (rank order); returns the list of
    per-rank results.  Used by the CPU tests of the carry logic; the arithmetic mirrors the device path:
    fp64 totals, fp64 carry, fp64 running value rounded to fp32 on store."""
    totals = []
    for s in shards:
        s64 = s.astype(np.float64)
        totals.append(np.sum(s64) if op == 'add' else np.prod(s64))
    results = []
    for r, s in enumerate(shards):
        carry = exclusive_carry(totals, r, op)
        s64 = s.astype(np.float64)
        run = np.cumsum(s64) + carry if op == 'add' else np.cumprod(s64) * carry
        results.append(run.astype(np.float32))
    return results
