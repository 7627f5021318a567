"""Evaluation of operator graphs on a B200: ``evaluate`` / ``profile`` with ``target_language='b200'``.

Counterpart of the reference's standalone runtime (opveclib/operator.py:2099-2335): build the operator graph of
the requested outputs, fuse it when ``opt_level >= 3``, compile each kernel (cached), and run the kernels in
dependency order.  Differences by design: tensors live in device memory owned by torch, kernels are launched
through the C-ABI launcher on torch's current stream, intermediates are released after their last use (the
reference keeps them all, operator.py:2329), and there is no CPU target - if the launcher library or a GPU is
missing the call fails.
"""
import os

import numpy as np

from . import compiler, launcher
from .fuse import merge_op_dag
from .local import logger, get_math_mode, math_mode
from .opgraph import build_op_dag

_programs = {}
_DRYRUN = 'OVL_B200_DRYRUN'
# How many times the number of blocks that fit on the device at once a grid may hold (see KernelPlan._passes):
# element-wise kernels, tile (transposed operand) kernels, reduction-loop kernels.
GRID_ROUNDS = int(os.environ.get('OVL_GRID_ROUNDS', '16'))
TILE_ROUNDS = int(os.environ.get('OVL_TILE_ROUNDS', '16'))
RED_ROUNDS = int(os.environ.get('OVL_RED_ROUNDS', '4'))
SCAN_ROUNDS = int(os.environ.get('OVL_SCAN_ROUNDS', '1'))


def _torch():
    import torch
    return torch


def warp_scan_shape(lines, sms):
    """(grid, block) of the warp-per-line scan (the same rule as ``ovl::warp_scan_shape`` of the templates): every
    warp walks whole lines one after the other, so among the residencies the kernel's registers allow - 12 to 21
    warps per SM as two to four blocks of four to eight warps - take the one that leaves the fewest warp slots idle
    in the final pass over the lines, and among equals (within 2 %) the one with the most warps."""
    if lines >= 32768:
        # tens of thousands of (then short) lines: one line per warp in blocks of four warps, handed out by the
        # hardware as earlier blocks finish
        return ((lines + 3) // 4, 128)
    best, pick = -1.0, (1, 32)
    for per_sm, warps in ((3, 7), (4, 5), (3, 6), (2, 8), (2, 7), (3, 5), (2, 6), (3, 4)):
        slots = sms * per_sm * warps
        rounds = (lines + slots - 1) // slots
        used = lines / float(rounds * slots)
        if used > best + 0.02:
            best = used
            pick = (max(1, min((lines + warps - 1) // warps, sms * per_sm)), warps * 32)
    return pick


class KernelPlan(object):
    """A compiled kernel with its launchable variants (generic / vectorised / scan / reduction), created on first
    use."""

    def __init__(self, kernel, math='exact'):
        self.kernel = kernel
        self.math = math
        self.cubin, self.meta = compiler.compile_kernel(kernel, math)
        self.name = self.meta['name']
        self.in_types = kernel.input_types
        self.out_types = kernel.output_types
        self._modules = {}
        self._variants = {}
        self._scratch = {}
        self._arrays = {}
        self._sms = {}
        self.last_variant = None
        self.launches = 0

    def _module(self, device):
        if device not in self._modules:
            self._modules[device] = launcher.Module(self.cubin)
        return self._modules[device]

    def _sm_count(self, device):
        if device not in self._sms:
            self._sms[device] = _torch().cuda.get_device_properties(device).multi_processor_count
        return self._sms[device]

    def _make(self, device, symbol, grid, block, use_in, use_out, aligns, scratch=0, zero=0, smem=0, cooperative=False):
        """A launchable kernel of this plan's module taking inputs[use_in] and outputs[use_out]."""
        key = (symbol, device)
        if key not in self._variants:
            types = [self.in_types[i] for i in use_in] + [self.out_types[i] for i in use_out]
            self._variants[key] = (launcher.Kernel(self._module(device), symbol, grid, block,
                                                   [t.dtype.code for t in types], [t.size for t in types], len(use_in),
                                                   aligns, scratch, zero, smem, cooperative), use_in, use_out)
        return self._variants[key]

    def _passes(self, which, device):
        """The launches that make up one execution of the chosen variant, in order."""
        meta = self.meta
        sms = self._sm_count(device)
        n_in, n_out = len(self.in_types), len(self.out_types)
        all_in, all_out = list(range(n_in)), list(range(n_out))
        if which in ('gen', 'vec'):
            m = meta[which]
            block = m['block']
            # up to GRID_ROUNDS times as many blocks as fit on the device at once: blocks that finish early make room
            # for new ones, so an SM whose warps ran ahead does not idle until the slowest block of a fixed
            # partition is done (a kernel that issues instructions most of the time gains 10 % over a grid of
            # exactly the resident blocks, a kernel limited by memory bandwidth 13 %)
            grid = max(1, min((m['items'] + block - 1) // block, sms * (2048 // block) * GRID_ROUNDS))
            aligns = [0] * (n_in + n_out)
            if which == 'vec':
                for kind, idx in m['aligned']:
                    aligns[idx if kind == 'in' else n_in + idx] = 16
            return [self._make(device, m['symbol'], grid, block, all_in, all_out, aligns)]
        if which == 'tile':
            m = meta['tile']
            grid = max(1, min(m['tiles'], sms * (2048 // m['block']) * TILE_ROUNDS))
            return [self._make(device, m['symbol'], grid, m['block'], all_in, all_out, [0] * (n_in + n_out))]
        if which == 'rows':
            m = meta['rows']
            per_sm = max(1, min(2048 // m['block'], (200 * 1024) // max(1, m['smem'])))
            grid = max(1, min((m['items'] + m['block'] - 1) // m['block'], sms * per_sm * GRID_ROUNDS))
            return [self._make(device, m['symbol'], grid, m['block'], all_in, all_out, [0] * (n_in + n_out), 0, 0,
                               m['smem'])]
        if which == 'red':
            m = meta['red']
            if m.get('split'):
                # few workers, long loops: enough slices per worker (or per group of 32 workers) for twice the blocks
                # that fit on the device at once (the hardware hands them out as earlier ones finish), each at least
                # split['slice'] trips long
                sp = m['split']
                per_sm = 2 * (2048 // m['block'])
                splits = max(1, min(sp['max'], (per_sm * sms + sp['units'] - 1) // sp['units'], m['trips'] // sp['slice']))
                return [self._make(device, m['symbol'], sp['units'] * splits, m['block'], all_in, all_out,
                                   [0] * (n_in + n_out), sp['scratch_bytes'], sp['zero_bytes'])]
            blocks = (m['items'] + m['workers_per_block'] - 1) // m['workers_per_block']
            grid = max(1, min(blocks, sms * (2048 // m['block']) * RED_ROUNDS))
            return [self._make(device, m['symbol'], grid, m['block'], all_in, all_out, [0] * (n_in + n_out))]
        m = meta['scan']
        block, name = m['block'], m['name']
        if which == 'cwalk':
            w = m['walk']
            # (one block per strip: with more strips than fit at once the hardware hands them out as blocks finish)
            return [self._make(device, w['symbol'], max(1, w['strips']), w['block'], [0], [0], [0, 0])]
        if which in ('cscan', 'cscanu'):
            suffix = '' if which == 'cscan' else 'u'
            al = 16 if which == 'cscan' else 0
            warps = block // 32
            tiles = m['tiles'][suffix]
            cap = sms * (2048 // block)
            scratch = m['scratch_bytes']
            return [self._make(device, name + '_cagg' + suffix, max(1, min((tiles + warps - 1) // warps, cap)), block, [0], [],
                               [al], scratch, m['zero_bytes']),
                    self._make(device, name + '_cpfx', max(1, min((m['columns'] + warps - 1) // warps, cap)), block, [], [],
                               [], scratch, 0),
                    self._make(device, name + '_cscan' + suffix, max(1, min((tiles + warps - 1) // warps, cap)), block, [0],
                               [0], [al, al], scratch, 0)]
        if which == 'wscan' and m['warp'].get('flat_vectors'):
            # short lines: a warp takes a chunk of whole lines per step, four warps per block
            grid = max(1, min((m['warp']['chunks'] + 3) // 4, sms * 128))
            return [self._make(device, m['warp']['symbol'], grid, m['warp']['block'], [0], [0], [16, 16])]
        if which == 'wscan':
            grid, block = warp_scan_shape(m['lines'], sms)

            return [self._make(device, m['warp']['symbol'], grid, block, [0], [0], [16, 16])]
        cap = sms * m['blocks_per_sm'] * SCAN_ROUNDS
        scratch = m['scratch_bytes']
        passes = []
        ring = m.get('ring')
        if which == 'ring':
            grid = max(1, min(m['tiles'], sms, ring['max_grid']))
            return [self._make(device, ring['symbol'], grid, ring['block'], [0], [0], [16, 16], scratch,
                               ring['zero_bytes'], ring['smem'], True)]
        suffix = '' if which == 'scan' else 'u'
        al = m['align_bytes'] if which == 'scan' else 0
        if m['three_pass']:
            passes.append(self._make(device, name + '_agg' + suffix, max(1, min(m['tiles'], cap)), block, [0], [], [al],
                                     scratch, m['zero_bytes']))
            passes.append(self._make(device, name + '_pfx', max(1, min(m['lines'], cap)), block, [], [], [], scratch, 0))
            passes.append(self._make(device, name + '_scan' + suffix, max(1, min(m['tiles'], cap)), block, [0], [0],
                                     [al, al], scratch, 0))
        else:
            passes.append(self._make(device, name + '_scan' + suffix, max(1, min(m['tiles'], cap)), block, [0], [0],
                                     [al, al], scratch, m['zero_bytes']))
        return passes

    def choose(self, in_ptrs, out_ptrs):
        meta = self.meta
        if meta.get('scan') and meta['scan'].get('strided'):
            if meta['scan'].get('walk') and os.environ.get('OVL_COLSCAN_MODE') != 'threepass':
                return 'cwalk'
            if meta['scan']['aligned_variant'] and all(p % 16 == 0 for p in in_ptrs + out_ptrs):
                return 'cscan'
            return 'cscanu'
        if meta.get('scan'):
            if (meta['scan'].get('warp') and all(p % 16 == 0 for p in in_ptrs + out_ptrs)
                    and os.environ.get('OVL_SCAN_MODE') not in ('threepass', 'block')):
                return 'wscan'
            al = meta['scan']['align_bytes']
            if (meta['scan'].get('ring') and all(p % 16 == 0 for p in in_ptrs + out_ptrs)
                    and os.environ.get('OVL_SCAN_MODE') != 'threepass'):
                return 'ring'
            # (lines too short for a block each are only scanned cooperatively by the warp kernel)
            if not meta['scan'].get('short'):
                if meta['scan']['aligned_variant'] and all(p % al == 0 for p in in_ptrs + out_ptrs):
                    return 'scan'
                return 'scanu'
        if meta.get('red'):
            # rows short enough to be staged whose length is not a whole number of warp-wide steps: the staged kernel
            # (a thread per row, rows read as one contiguous piece) beats a warp per row with a ragged last step
            # (fp32 rows of 200: 5.0 against 4.2 TB/s; rows of 128, 160, 256: the warp per row wins, 5.8 - 6.0 against
            # 4.2 - 5.3)
            if (meta.get('rows') and meta['red'].get('group') == 32 and meta['red']['trips'] % 32
                    and os.environ.get('OVL_ROWS_MODE') != 'off'):
                return 'rows'
            return 'red'
        if meta.get('tile') and os.environ.get('OVL_TILE_MODE') != 'off':
            return 'tile'
        if meta.get('rows') and os.environ.get('OVL_ROWS_MODE') != 'off':
            return 'rows'
        if meta.get('vec'):
            ok = True
            for kind, idx in meta['vec']['aligned']:
                p = in_ptrs[idx] if kind == 'in' else out_ptrs[idx]
                if p % 16 != 0:
                    ok = False
            if ok:
                return 'vec'
        return 'gen'

    def launch(self, ins, outs, stream_ptr, device, iterations=None):
        """ins/outs: torch CUDA tensors.  Enqueues one execution (or ``iterations`` timed ones, returning the
        milliseconds of each, summed over the passes of a multi-pass kernel)."""
        torch = _torch()
        in_ptrs = [t.data_ptr() for t in ins]
        out_ptrs = [t.data_ptr() for t in outs]
        which = self.choose(in_ptrs, out_ptrs)
        passes = self._passes(which, device)
        self.last_variant = which
        scratch_ptr, scratch_bytes = None, 0
        need = max(k.scratch_bytes for k, _, _ in passes)
        if need:
            key = (device, stream_ptr)
            buf = self._scratch.get(key)
            if buf is None or buf.numel() < need:
                buf = torch.empty(need, dtype=torch.uint8, device='cuda:%d' % device)
                self._scratch[key] = buf
            scratch_ptr, scratch_bytes = buf.data_ptr(), buf.numel()
        # A multi-pass kernel is timed one whole pass sequence per iteration: the middle pass of a three-pass scan
        # turns the tile aggregates into prefixes in place, so repeating it alone would feed it its own output.
        rounds = [None] if iterations is None else ([iterations] if len(passes) == 1 else [1] * iterations)
        total_ms = None if iterations is None else []
        for count in rounds:
            round_ms = None
            for pi, (k, use_in, use_out) in enumerate(passes):
                akey = (which, pi, tuple(in_ptrs), tuple(out_ptrs))
                arrays = self._arrays.get(akey)
                if arrays is None:
                    if len(self._arrays) > 64:
                        self._arrays.clear()
                    arrays = (launcher.tensor_array([(in_ptrs[i], self.in_types[i].dtype.code, self.in_types[i].size)
                                                     for i in use_in]),
                              launcher.tensor_array([(out_ptrs[i], self.out_types[i].dtype.code, self.out_types[i].size)
                                                     for i in use_out]))
                    self._arrays[akey] = arrays
                in_arr, out_arr = arrays
                sp, sb = (scratch_ptr, scratch_bytes) if k.scratch_bytes else (None, 0)
                if count is None:
                    st = k.launch(in_arr, len(use_in), out_arr, len(use_out), sp, sb, stream_ptr)
                    launcher.check(st, 'launching ' + self.kernel.name)
                    self.launches += 1
                else:
                    st, ms = k.profile(in_arr, len(use_in), out_arr, len(use_out), sp, sb, stream_ptr, count)
                    launcher.check(st, 'profiling ' + self.kernel.name)
                    self.launches += count
                    round_ms = list(ms) if round_ms is None else [a + b for a, b in zip(round_ms, ms)]
            if count is not None:
                total_ms.extend(round_ms)
        return total_ms

    def check_status(self, stream_ptr, device):
        """Raise if a bounded device-side wait of this kernel expired (scan kernels only).  Looks at the scratch
        buffer of every stream the kernel ran on, on this device."""
        import ctypes
        for (dev, _), buf in list(self._scratch.items()):
            if dev != device:
                continue
            status = ctypes.c_int32(0)
            launcher.check(launcher.library().ovl_read_kernel_status(buf.data_ptr(), stream_ptr, ctypes.byref(status)),
                           'reading kernel status')
            if status.value != 0:
                raise launcher.OvlError(status.value, 'kernel ' + self.kernel.name)


class Program(object):
    """A compiled operator graph: kernel plans in launch order plus the wiring between them."""

    def __init__(self, dag, math='exact'):
        self.dag = dag
        self.math = math
        self.plans = [KernelPlan(k, math) for k in dag.kernels]
        # last consumer of every intermediate, so its memory can be released early
        self.last_use = {}
        for op_index, refs in enumerate(dag.references):
            for r in refs:
                if not r.is_leaf:
                    self.last_use[(r.op_index, r.op_output_index)] = op_index
        self.keep = set(dag.outputs)

    def run(self, leaf_tensors, device, stream_ptr, iterations=None, out_buffers=None):
        """leaf_tensors: torch CUDA tensors for the graph inputs.  Returns (outputs, {name: ms list})."""
        torch = _torch()
        buffers = {}
        times = {}
        for op_index, plan in enumerate(self.plans):
            ins = []
            for r in self.dag.references[op_index]:
                ins.append(leaf_tensors[r.dag_input_index] if r.is_leaf else buffers[(r.op_index, r.op_output_index)])
            outs = []
            for k, t in enumerate(plan.out_types):
                preset = None
                if out_buffers is not None and (op_index, k) in self.keep:
                    preset = out_buffers[self.dag.outputs.index((op_index, k))]
                if preset is None:
                    preset = torch.empty(t.shape, dtype=t.dtype.as_torch(), device='cuda:%d' % device)
                outs.append(preset)
                buffers[(op_index, k)] = preset
            ms = plan.launch(ins, outs, stream_ptr, device, iterations)
            if ms is not None:
                times[plan.name] = np.array(ms, dtype=np.float64)
            for key in [key for key, last in self.last_use.items() if last == op_index and key not in self.keep]:
                buffers.pop(key, None)
        return [buffers[o] for o in self.dag.outputs], times

    def capture(self, leaf_tensors, device, out_buffers):
        """Record one execution of the graph into a CUDA graph (``torch.cuda.CUDAGraph``) over fixed input and
        output tensors; ``replay()`` then costs one launch call whatever the number of kernels.  For loops whose
        kernels are shorter than the time it takes to enqueue them."""
        torch = _torch()
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            # first run outside the capture: loads modules, creates kernels and this stream's scratch buffers
            self.run(leaf_tensors, device, side.cuda_stream, None, out_buffers)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            self.run(leaf_tensors, device, side.cuda_stream, None, out_buffers)
        return graph

    def check_status(self, device, stream_ptr):
        for plan in self.plans:
            if plan.meta.get('scan'):
                plan.check_status(stream_ptr, device)


_host_scans = {}
_HOST_SCAN_CHUNK = 1 << 26
_HOST_SCAN_MIN = 1 << 25


def _host_scan_plan(prog):
    """('add' | 'mul', n) when the program is one scan of a single long fp32 line (the chunk-pipelined host path
    handles exactly that), else None."""
    if len(prog.plans) != 1 or len(prog.dag.outputs) != 1:
        return None
    plan = prog.plans[0]
    m = plan.meta.get('scan')
    if not m or m.get('strided') or m['lines'] != 1 or m['n'] < _HOST_SCAN_MIN:
        return None
    if plan.in_types[0].dtype.name != 'float32' or len(plan.in_types) != 1:
        return None
    return m['op'], m['n']


def as_output_list(outputs):
    """The outputs behind what a caller handed to ``evaluate``: a list or tuple is taken as it is; a single
    operator stands for all of its outputs (the reference unpacks it the same way,
    opveclib/operator.py:2256: ``_build_op_dag(*output_list)`` iterates an operator); one output is itself."""
    from .opgraph import Operator
    if isinstance(outputs, (list, tuple)):
        return list(outputs)
    if isinstance(outputs, Operator) and len(outputs) > 1:
        return list(outputs)
    return [outputs]


def compile_outputs(output_list, opt_level=3, math=None):
    """Build, fuse and compile the operator graph behind ``output_list``; cached by graph structure and math
    lowering (``math=None``: the current mode, :func:`opveclib_b200.local.get_math_mode`)."""
    output_list = as_output_list(output_list)
    dag = build_op_dag(*output_list)
    math = math or get_math_mode()
    key = (dag.text(), opt_level >= 3, math)
    prog = _programs.get(key)
    if prog is None:
        fused = merge_op_dag(dag) if opt_level >= 3 else dag
        prog = Program(fused, math)
        _programs[key] = prog
    return prog, dag


def _is_torch(x):
    return type(x).__module__.startswith('torch')


def profile(output_list, target_language='b200', profiling_iterations=1, opt_level=3, out=None, math=None):
    """Evaluate operator outputs.  Returns (list of results, {kernel name: ms per iteration}).

    ``math`` (extension): 'exact' or 'tolerance' for this call; None takes the current mode (``ovl.math_mode``,
    ``ovl.set_math_mode``, environment variable OVL_B200_MATH; 'exact' unless changed).

    ``out`` (extension): a list with one preallocated numpy array per requested output (pinned host memory
    makes the copy back asynchronous and fast); results are written there instead of into fresh arrays.

    Leaf inputs may be numpy arrays (staged to the device and results copied back, as the reference harness
    does at opveclib/testcudaop.cc:84-183, 306-379) or torch tensors; with any torch CUDA input the results stay
    on the device as torch tensors."""
    if target_language not in ('b200', 'cuda'):
        raise ValueError('Unsupported target_language: ' + str(target_language) +
                         " (this backend runs on the GPU only: use 'b200')")
    if not isinstance(profiling_iterations, int) or profiling_iterations < 1:
        raise ValueError('profiling_iterations must be a positive int')
    with math_mode(math):
        return _profile(output_list, profiling_iterations, opt_level, out)


def _profile(output_list, profiling_iterations, opt_level, out):
    prog, dag = compile_outputs(output_list, opt_level)
    if os.environ.get(_DRYRUN):
        # cache-warming mode for machines without a GPU: everything is compiled, nothing is launched
        return [np.zeros(dag.kernels[o].output_types[k].shape, dtype=dag.kernels[o].output_types[k].dtype.as_numpy())
                for o, k in dag.outputs], {}
    torch = _torch()
    if not torch.cuda.is_available():
        raise RuntimeError('opveclib_b200 needs a CUDA device: there is no CPU execution path')
    device = torch.cuda.current_device()
    any_cuda_input = False
    leaves = []
    for x, t in zip(dag.inputs, dag.input_types):
        if _is_torch(x):
            if x.is_cuda:
                any_cuda_input = True
                device = x.device.index
            leaves.append(x)
        else:
            leaves.append(torch.from_numpy(np.ascontiguousarray(x)))
    dev = 'cuda:%d' % device
    if not any(_is_torch(x) for x in dag.inputs) and profiling_iterations == 1:
        # a host-resident long fp32 line that is scanned: chunks stream through the device, both link directions busy
        hs = _host_scan_plan(prog)
        if hs is not None:
            op, n = hs
            shape = tuple(prog.plans[0].out_types[0].shape)
            dst = out[0] if out is not None else np.empty(shape, dtype=np.float32)
            if dst.shape != shape or dst.dtype != np.float32 or not dst.flags['C_CONTIGUOUS']:
                raise ValueError('out must hold one C-contiguous array of the right shape and dtype per output')
            key = (op, device)
            if key not in _host_scans:
                from . import parallel
                with torch.cuda.device(device):
                    _host_scans[key] = parallel.HostScan(_HOST_SCAN_CHUNK, op)
            src = np.ascontiguousarray(dag.inputs[0]).reshape(-1)
            with torch.cuda.device(device):
                _host_scans[key](torch.from_numpy(src), torch.from_numpy(dst.reshape(-1)))
            return [dst], {prog.plans[0].name: np.array([np.nan])}
        # host-resident inputs: stream slabs of rows through the device when the graph allows it
        from . import streaming
        splan = streaming.plan(as_output_list(output_list), dag, prog,
                               opt_level)
        if splan is not None:
            out_types = [prog.plans[o].out_types[k] for o, k in prog.dag.outputs]
            if out is None:
                host_out = [np.empty(t.shape, dtype=t.dtype.as_numpy()) for t in out_types]
            else:
                host_out = list(out)
                if len(host_out) != len(out_types) or any(
                        a.shape != tuple(t.shape) or a.dtype != t.dtype.as_numpy() or not a.flags['C_CONTIGUOUS']
                        for a, t in zip(host_out, out_types)):
                    raise ValueError('out must hold one C-contiguous array of the right shape and dtype per output')
            host_in = [np.ascontiguousarray(x) for x in dag.inputs]
            streaming.run(splan, host_in, host_out, out_types, device)
            return host_out, {plan.name: np.array([np.nan]) for plan in splan['prog'].plans}
    with torch.cuda.device(device):
        stream_ptr = torch.cuda.current_stream().cuda_stream
        staged = [x.contiguous() if x.is_cuda else x.to(dev, non_blocking=True) for x in leaves]
        if profiling_iterations == 1 and not logger.isEnabledFor(10):
            outs, times = prog.run(staged, device, stream_ptr, None)
            for plan in prog.plans:
                times[plan.name] = np.array([np.nan])
        else:
            outs, times = prog.run(staged, device, stream_ptr, profiling_iterations)
        if any_cuda_input:
            prog.check_status(device, stream_ptr)
            return outs, times
        if out is not None:
            if len(out) != len(outs):
                raise ValueError('out must hold one array per requested output')
            host = []
            for dst, o in zip(out, outs):
                if dst.shape != tuple(o.shape) or not dst.flags['C_CONTIGUOUS'] or \
                        dst.dtype.name != str(o.dtype).replace('torch.', ''):
                    raise ValueError('out array has the wrong shape, dtype or layout')
                torch.from_numpy(dst).copy_(o, non_blocking=True)
                host.append(dst)
            torch.cuda.current_stream().synchronize()
        else:
            host = [o.cpu().numpy() for o in outs]
        prog.check_status(device, stream_ptr)
    return host, times


def evaluate(output_list, target_language='b200', opt_level=3, out=None, math=None):
    """Evaluate operator outputs on the GPU; a single output comes back bare, several as a list
    (opveclib/operator.py:2099-2117).  ``math``: see :func:`profile`."""
    outs, _ = profile(output_list, target_language=target_language, profiling_iterations=1, opt_level=opt_level,
                      out=out, math=math)
    return outs[0] if len(outs) == 1 else outs
