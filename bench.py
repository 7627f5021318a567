"""Benchmark of the hot path: fused OVL operator graphs on B200, next to the reference's CPU operator.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--math tolerance|exact]
                    [--workload c4|c5|c2_cumsum|c2_cumprod|c1|c1_shift|c3|c3_grad|c3_stdops|light16|matvec|perf_accumulate|colscan|colscan_wide|colsum|colsum_narrow|dot_long|rowsum_short|rownorm_short|scan_tiny|rows_short|transpose|transpose_axpy|op_<name>]

Default workload (the one the headline metric is quoted on): the 16-operator fused element-wise chain over an
fp32 tensor [8, 2^27] drawn from uniform[-2, 2], rows sharded contiguously over N GPUs with no communication
(total work fixed: strong scaling).  One step is one evaluation of the whole operator graph on the rank's rows.
Kernels are generated with the math lowering named in ``config.math`` (default 'tolerance': fp32 division, exp, log
and tanh with bounded error - the counterpart of the reference's own CUDA build, which uses --use_fast_math,
opveclib/operator.py:2081); the default run also times the 'exact' lowering and reports it as ``exact_math``.
After the headline workload the default run times the scan across shard boundaries (`c5`, fp32 [2^31] split over the
same N GPUs, totals exchanged through peer memory or a collective) and reports it as ``secondary.c5``.
The other workloads exist for profiling single kernels: `c5` is the scan across shard boundaries, `matvec` a
per-row reduction loop, `dot_long` / `colsum_narrow` reduction loops of very few workers (one dot product of 2^28 terms,
column sums of [2^22, 64]: the loop is cut into slices for many blocks), `perf_accumulate` the reference's own timing harness (fp64 [10000, 1000] cumsum along axis 0),
`colscan` a column scan far larger than L2, `transpose` / `transpose_axpy` an operand read along the workgroup's
first axis, `op_<name>` one operator of the chain on its own.

Prints one JSON line (rank 0).  ``value`` is elements/s with inputs resident in HBM, timed with CUDA events on
the launching stream, maximum over ranks; ``e2e`` is the same work through ``ovl.evaluate`` from pinned host
arrays and back (host<->device copies inside the timed region); ``roofline`` relates the dominant kernel's
algorithmic bytes per launch to the measured HBM copy bandwidth (and, as ``same_size_copy_ms``, to a plain device copy
of the same number of bytes timed the same way - what that peak becomes at the workload's own size); ``cpu_baseline`` times the reference's own
generated C++ operators (oracle/_ref, else the oracle port) on this machine's host cores over a bounded sample.
``--impl reference`` runs only that CPU arm and prints it in the same format.
"""
import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

C4_ROWS, C4_COLS = 8, 1 << 27
C4_SAMPLE_COLS = 1 << 24          # CPU sample: one row of 2^24 elements (1/64 of the workload)
C5_TOTAL = 1 << 31
C5_SAMPLE = 1 << 26
SEED = 1234
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


# ---------------------------------------------------------------------------------------------------------
def measured_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    try:
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    except Exception:
        return FALLBACK_HBM_GBS, 'fallback'


def profiled_traffic(workload, elements_per_launch):
    """DRAM bytes per launch scaled from the committed ncu summary (bytes per element), or None."""
    path = os.path.join(ROOT, 'profiles', workload + '_kernel.md')
    try:
        with open(path) as f:
            m = re.search(r'dram_bytes_per_element:\s*([0-9.]+)', f.read())
        return float(m.group(1)) * elements_per_launch if m else None
    except Exception:
        return None


class ClockSampler(object):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.gpu), '--query-gpu=' + self.FIELDS,
                                          '--format=csv,noheader,nounits', '-lms', '100'], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, universal_newlines=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in self.lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith('active'):
                    reasons.add(n)
        busy = [c for c in sm if c > 0.5 * (mx or 1)] or sm
        return {'sm_mhz': float(np.median(busy)) if busy else None, 'sm_max_mhz': mx, 'reasons': sorted(reasons),
                'samples': len(sm)}


# ---------------------------------------------------------------------------------------------------------
def dist_env():
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    return rank, world, local


def build_graph(workload, rows_local=None, n_local=None):
    """(operator outputs, input shapes, elements per step on this rank, algorithmic bytes per element)."""
    from opveclib_b200.examples import workloads as cases
    ns = cases.namespace()
    f32 = np.float32
    z = lambda *shape: np.zeros(shape, dtype=f32)     # noqa: E731  (only the type matters for tracing)
    if workload == 'c4':
        return [cases.chain16(ns, z(rows_local, C4_COLS))], rows_local * C4_COLS, 8
    if workload == 'light16':
        return [cases.chain16_light(ns, z(rows_local or C4_ROWS, C4_COLS))], (rows_local or C4_ROWS) * C4_COLS, 8
    if workload == 'c2_cumsum':
        return [ns.cumsum(z(4096, 8192), axis=1)], 4096 * 8192, 8
    if workload == 'c2_cumprod':
        return [ns.cumprod(z(4096, 8192), axis=1)], 4096 * 8192, 8
    if workload == 'c1':
        return [cases.c1_chain(ns, z(1 << 20))], 1 << 20, 8
    if workload == 'c1_shift':
        return [cases.user_ops(ns).shift_cyclic(z(1 << 20))], 1 << 20, 8
    if workload == 'c3':
        op = ns.lstm(z(512, 4096), z(512, 1024), forget_bias=0.0)
        return [op[0], op[1]], 512 * 1024, 28
    if workload == 'c3_grad':
        op = ns.lstm_grad(z(512, 4096), z(512, 1024), z(512, 1024), z(512, 1024), forget_bias=0.0)
        return [op[0], op[1]], 512 * 1024, 48
    if workload == 'c3_stdops':
        # the same cell composed from the operator library (split -> sigmoid / tanh -> mul -> add; the graph of
        # opveclib/test/test_operator_merge.py:311-321): fusion must turn it into the hand-fused cell's one kernel
        return cases.stdops_lstm(ns, z(512, 4096), z(512, 1024)), 512 * 1024, 28
    if workload.startswith('op_'):
        # one operator of the 16-operator chain on its own (instruction cost per element), fp32 [1, 2^26]
        u = cases.user_ops(ns)
        x = z(1, 1 << 26)
        single = {'op_tanh': lambda: u.ew_tanh(x), 'op_exp': lambda: u.ew_exp(x), 'op_log1p': lambda: ns.log1p(x),
                  'op_expm1': lambda: ns.expm1(x), 'op_mulc': lambda: u.ew_mulc(x, c=0.5), 'op_add': lambda: u.ew_add(x, x),
                  'op_where': lambda: u.where_greater(x, x)}
        return [single[workload]()], 1 << 26, 8
    if workload == 'perf_accumulate':
        # the reference's own timing harness: cumsum of fp64 [10000, 1000] along axis 0
        # (opveclib/examples/test_perf_accumulate.py:35-48); 8 B read + 8 B written per element
        return [ns.cumsum(np.zeros((10000, 1000), dtype=np.float64), axis=0)], 10000 * 1000, 16
    if workload == 'colscan':
        # a column scan far larger than L2: cumsum of fp32 [32768, 8192] along axis 0 (1 GiB in, 1 GiB out)
        return [ns.cumsum(z(32768, 8192), axis=0)], 32768 * 8192, 8
    if workload == 'colscan_wide':
        # more strips of columns than blocks fit on the device: cumsum of fp32 [8192, 32768] along axis 0
        return [ns.cumsum(z(8192, 32768), axis=0)], 8192 * 32768, 8
    if workload == 'colsum':
        # column sums as a per-column reduction loop over the rows of fp32 [16384, 8192]: the matrix is read once
        return [cases.user_ops(ns).colsum(z(16384, 8192))], 16384 * 8192, 4
    if workload == 'rows_short':
        # many short lines: cumsum along axis 1 of fp32 [131072, 512] (256 MiB in, 256 MiB out), a warp per line
        return [ns.cumsum(z(131072, 512), axis=1)], 131072 * 512, 8
    if workload == 'transpose':
        # an operand read along the workgroup's first axis: fp32 [16384, 16384] -> its transpose (1 GiB in, 1 GiB out)
        return [cases.user_ops(ns).transpose(z(16384, 16384))], 16384 * 16384, 8
    if workload == 'transpose_axpy':
        # out = a^T * 0.5 + b: one transposed operand fused with a straight one, 12 B per element
        return [cases.user_ops(ns).transpose_axpy(z(16384, 16384), z(16384, 16384), alpha=0.5)], 16384 * 16384, 12
    if workload == 'matvec':
        # reduction loop per row (documentation/programming.rst:320-344): the matrix is read once, 4 B per element
        return [cases.user_ops(ns).matvec(z(16384, 8192), z(8192))], 16384 * 8192, 4
    if workload == 'dot_long':
        # ONE dot product of 2^28 terms (matvec with a single row): the loop is cut into slices that many blocks
        # fold; 1 GiB + 1 GiB, every element read once
        return [cases.user_ops(ns).matvec(z(1, 1 << 28), z(1 << 28))], 2 << 28, 4
    if workload == 'rowsum_short':
        # row sums of fp32 [2^22, 32]: the rows of a block's workers staged in shared memory, summed in order
        return [cases.user_ops(ns).rowsum(z(1 << 22, 32))], 32 << 22, 4
    if workload == 'rownorm_short':
        # every row of fp32 [2^21, 50] divided by its sum: input and output rows through shared memory, 8 B per element
        return [cases.user_ops(ns).row_normalise(z(1 << 21, 50))], 50 << 21, 8
    if workload == 'scan_tiny':
        # cumsum along axis 1 of fp32 [2^20, 128]: short lines share warps, the tensor streamed as one flat array
        return [ns.cumsum(z(1 << 20, 128), axis=1)], 128 << 20, 8
    if workload == 'colsum_narrow':
        # column sums of fp32 [2^22, 64]: two groups of 32 columns, the rows cut into slices for many blocks
        return [cases.user_ops(ns).colsum(z(1 << 22, 64))], 64 << 22, 4
    raise ValueError('unknown workload ' + workload)


def precompile():
    """Compile the kernels of every benchmark workload (no GPU needed)."""
    from opveclib_b200 import runtime, streaming
    from opveclib_b200.local import math_mode
    for math in ('tolerance', 'exact'):
        with math_mode(math):
            _precompile_all(runtime, streaming)


def _precompile_all(runtime, streaming):
    for n in (1, 2, 4, 8):
        outs = build_graph('c4', rows_local=C4_ROWS // n)[0]
        prog, dag = runtime.compile_outputs(outs)
        streaming.plan(outs, dag, prog, 3)          # the slab-shaped kernels of the end-to-end leg
    for w in ('c2_cumsum', 'c2_cumprod', 'c1', 'c1_shift', 'c3', 'c3_grad', 'c3_stdops', 'light16', 'matvec', 'op_tanh', 'op_exp',
              'op_log1p', 'op_expm1', 'op_mulc', 'op_add', 'op_where', 'perf_accumulate', 'colscan', 'colscan_wide', 'transpose',
              'transpose_axpy', 'rows_short', 'colsum', 'dot_long', 'colsum_narrow', 'rowsum_short', 'rownorm_short',
              'scan_tiny'):
        runtime.compile_outputs(build_graph(w)[0])


def input_distribution(workload, index):
    if workload in ('c4', 'light16') or workload.startswith('op_'):
        return ('uniform', -2.0, 2.0)
    if workload == 'c2_cumprod':
        return ('uniform', 0.99, 1.01)
    if workload in ('c1', 'c1_shift'):
        return ('uniform', -1.0, 1.0)
    if workload in ('perf_accumulate', 'rownorm_short'):
        return ('uniform', 0.5, 1.5) if workload == 'rownorm_short' else ('uniform', 0.0, 1.0)
    if workload == 'c3_grad' and index >= 2:
        return ('normal', 0.0, 0.1)
    return ('normal', 0.0, 1.0)


def make_device_inputs(torch, workload, types, device, seed):
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = []
    for i, t in enumerate(types):
        kind, a, b = input_distribution(workload, i)
        x = torch.empty(t.shape, dtype=t.dtype.as_torch(), device=device)
        if kind == 'uniform':
            x.uniform_(a, b, generator=gen)
        else:
            x.normal_(a, b, generator=gen)
        out.append(x)
    return out


# ---------------------------------------------------------------------------------------------------------
def cpu_reference_run(workload, iterations):
    """Time the reference's CPU implementation on a bounded sample.  Returns a dict for ``cpu_baseline``."""
    from oracle import ref_runner, runner
    from opveclib_b200.examples import workloads as cases
    rs = np.random.RandomState(SEED)
    if workload == 'c4':
        name, shape, sample = 'c4_chain16_1x%d' % C4_SAMPLE_COLS, (1, C4_SAMPLE_COLS), \
            'one row slice [1, 2^24] of the [8, 2^27] tensor (1/64 of a step)'
        inputs = [rs.uniform(-2, 2, shape).astype(np.float32)]
        elements = C4_SAMPLE_COLS
    elif workload == 'c5':
        name, shape, sample = 'c5_cumsum_%d' % C5_SAMPLE, (C5_SAMPLE,), 'first 2^26 of 2^31 elements (1/32 of a step)'
        inputs = [rs.normal(0, 1, shape).astype(np.float32)]
        elements = C5_SAMPLE
    else:
        table = {'c2_cumsum': 'c2_cumsum_4096x8192', 'c2_cumprod': 'c2_cumprod_4096x8192', 'c1': 'c1_chain_1048576',
                 'c1_shift': 'c1_shift_1048576', 'c3': 'c3_lstm_512x1024', 'c3_grad': 'c3_lstm_grad_512x1024'}
        name, sample = table.get(workload, workload), 'the full workload'
        outs, elements, _ = build_graph(workload)
        from opveclib_b200.opgraph import build_op_dag
        types = build_op_dag(*outs).input_types
        inputs = []
        for i, t in enumerate(types):
            kind, a, b = input_distribution(workload, i)
            inputs.append((rs.uniform(a, b, t.shape) if kind == 'uniform' else rs.normal(a, b, t.shape)).astype(t.dtype.as_numpy()))
    if ref_runner.available(name):
        threads = ref_runner.hardware_threads()
        _, ms = ref_runner.run(name, inputs, num_threads=0, variant='opt', iterations=iterations)
        _, ms_ref = ref_runner.run(name, inputs, num_threads=0, variant='ref', iterations=1)
        kind = 'reference'
        extra = {'ms_reference_flags': float(ms_ref.min()), 'ops_after_reference_merge':
                 len(ref_runner.manifest()[name]['ops'])}
    else:
        # the oracle port: same generated arithmetic from this repository's restatement of the generator
        ns = cases.namespace()
        if workload == 'c4':
            outs = [cases.chain16(ns, inputs[0])]
        elif workload == 'c5':
            outs = [ns.cumsum(inputs[0])]
        else:
            outs = rebuild_with_inputs(workload, inputs, None)
        threads = runner.hardware_threads()
        _, times = runner.profile(outs, num_threads=0, iterations=iterations)
        ms = sum(times.values())
        kind, extra = 'port', {}
    single_threaded = workload == 'c5'   # a rank-1 accumulate is one worker (test_accumulate.py:40-41)
    best = float(np.min(ms))
    res = {'value': elements / (best * 1e-3), 'unit': 'elements/s', 'cores': 1 if single_threaded else threads,
           'kind': kind, 'sample': sample, 'ms_per_sample': best, 'ms_per_sample_median': float(np.median(ms)),
           'iterations': int(np.size(ms)), 'build': '-O2 -ffp-contract=off'}
    res.update(extra)
    return res, elements


def run_reference_arm(args, workload):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    t0 = time.time()
    base, elements = cpu_reference_run(workload, max(1, args.warmup))   # warm-up passes
    res, elements = cpu_reference_run(workload, max(1, args.steps))
    line = {
        'impl': 'reference', 'metric': 'fused-op elements/s', 'value': res['value'], 'unit': 'elements/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': res['ms_per_sample'],
        'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f64' if workload == 'perf_accumulate' else 'f32',
        'data': 'synthetic', 'config': workload_config(workload, args.gpus), 'cpu_baseline': res,
        'e2e': {'value': res['value'], 'unit': 'elements/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0, 'wall_s': time.time() - t0,
    }
    print(json.dumps(line))
    return 0


def workload_config(workload, n):
    names = {
        'c4': 'fused 16-op element-wise chain, fp32 [8, 2^27] uniform[-2,2], rows sharded over the GPUs',
        'light16': 'fused 16-op element-wise chain without transcendentals (add/mul/where), fp32 [8, 2^27]',
        'c2_cumsum': 'cumsum along axis 1, fp32 [4096, 8192] normal(0,1)',
        'c2_cumprod': 'cumprod along axis 1, fp32 [4096, 8192] uniform[0.99,1.01]',
        'c1': 'fused chain expm1(log1p(|x|))*0.5+x, fp32 [2^20] uniform[-1,1]',
        'c1_shift': 'shift_cyclic by +1, fp32 [2^20]',
        'c3': 'LSTM cell forward, gates fp32 [512, 4096], c [512, 1024]',
        'c3_grad': 'LSTM cell gradient, gates fp32 [512, 4096], c/dc/dh [512, 1024]',
        'c3_stdops': 'LSTM cell forward composed from the operator library (split, sigmoid, tanh, mul, add), fused',
        'c5': 'cumsum along the sharded axis, fp32 [2^31] normal(0,1), contiguous shards, fp64 carry exchange',
        'matvec': 'matrix-vector product as a per-row reduction loop, fp32 [16384, 8192] x [8192] normal(0,1)',
        'perf_accumulate': "cumsum along axis 0, fp64 [10000, 1000] uniform[0,1] (the reference's own timing harness)",
        'colscan': 'cumsum along axis 0, fp32 [32768, 8192] normal(0,1)',
        'colscan_wide': 'cumsum along axis 0, fp32 [8192, 32768] normal(0,1)',
        'rows_short': 'cumsum along axis 1, fp32 [131072, 512] normal(0,1)',
        'colsum': 'column sums as a per-column reduction loop, fp32 [16384, 8192] normal(0,1)',
        'dot_long': 'one dot product of 2^28 terms (matvec fp32 [1, 2^28] x [2^28]), the loop split over the blocks',
        'colsum_narrow': 'column sums of fp32 [2^22, 64] normal(0,1), rows split over the blocks',
        'rowsum_short': 'row sums of fp32 [2^22, 32] normal(0,1), rows staged in shared memory',
        'rownorm_short': 'rows of fp32 [2^21, 50] uniform(0.5,1.5) divided by their sums, rows staged in shared memory both ways',
        'scan_tiny': 'cumsum along axis 1 of fp32 [2^20, 128] normal(0,1), several lines per warp',
        'transpose': 'transpose of fp32 [16384, 16384] normal(0,1) written as an operator that reads its operand transposed',
        'transpose_axpy': 'a^T * 0.5 + b, fp32 [16384, 16384] normal(0,1)',
    }
    if workload.startswith('op_'):
        names[workload] = 'single operator ' + workload[3:] + ' of the 16-operator chain, fp32 [1, 2^26] uniform[-2,2]'
    if workload == 'c5' and C5_TOTAL != 1 << 31:
        names['c5'] = 'cumsum along the sharded axis, fp32 [%d] normal(0,1) (reduced case)' % C5_TOTAL
    if workload == 'c4' and (C4_ROWS, C4_COLS) != (8, 1 << 27):
        names['c4'] = 'fused 16-op element-wise chain, fp32 [%d, %d] uniform[-2,2] (reduced case)' % (C4_ROWS, C4_COLS)
    return {'workload': names[workload], 'id': workload, 'parallelism': 'shard-leading-axis x%d' % n,
            'l2': 'inputs larger than L2 (126 MB)' if (workload in ('c4', 'light16', 'c5', 'c2_cumsum', 'c2_cumprod', 'matvec', 'colscan', 'colscan_wide', 'colsum', 'rows_short', 'transpose', 'transpose_axpy', 'dot_long', 'colsum_narrow', 'rowsum_short', 'rownorm_short', 'scan_tiny')
                                                      or workload.startswith('op_'))
            else 'inputs fit in L2; an L2-sized buffer is written between timed steps', 'seed': SEED}


# ---------------------------------------------------------------------------------------------------------
def bind_near_gpu(local):
    """Run this process (and so its first-touched and pinned host memory) on the CPUs of the GPU's NUMA node when
    the box has several nodes and the process is allowed on those CPUs.  Returns what was done, for the report."""
    info = {'numa_nodes': None, 'gpu_node': None, 'bound': False}
    try:
        import torch
        nodes = [d for d in os.listdir('/sys/devices/system/node') if re.match(r'node\d+$', d)]
        info['numa_nodes'] = len(nodes)
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        dom = torch.cuda.get_device_properties(local).pci_domain_id
        dev = torch.cuda.get_device_properties(local).pci_device_id
        path = '/sys/bus/pci/devices/%04x:%02x:%02x.0/numa_node' % (dom, bus, dev)
        with open(path) as f:
            node = int(f.read().strip())
        info['gpu_node'] = node
        if len(nodes) < 2 or node < 0:
            return info
        with open('/sys/devices/system/node/node%d/cpulist' % node) as f:
            cpus = set()
            for part in f.read().strip().split(','):
                lo, _, hi = part.partition('-')
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if allowed:
            os.sched_setaffinity(0, allowed)
            info['bound'] = True
            info['cpus'] = len(allowed)
    except Exception as exc:
        info['note'] = '%s: %s' % (type(exc).__name__, exc)
    return info


def time_steps(torch, step, steps, flush, barrier):
    """Milliseconds for ``steps`` steps on the current stream, CUDA events, barrier on both sides."""
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    barrier()
    if flush is None:
        start.record()
        for _ in range(steps):
            step()
        stop.record()
        barrier()
        return start.elapsed_time(stop)
    # L2-resident inputs: overwrite an L2-sized buffer between steps and time each step on its own
    total = 0.0
    for _ in range(steps):
        flush.fill_(1)
        start.record()
        step()
        stop.record()
        stop.synchronize()
        total += start.elapsed_time(stop)
    barrier()
    return total


def run_c5(torch, dist, parallel, args, rank, world, device, barrier, steps, warmup, with_e2e):
    """The scan across shard boundaries: fp32 [C5_TOTAL] split contiguously over the ranks.  Returns the report
    (rank 0) with ms_per_step as the maximum over ranks."""
    n_local = C5_TOTAL // world
    scan = parallel.ShardedScan(n_local, 'add', exchange=args.exchange)
    gen = torch.Generator(device=device)
    gen.manual_seed(SEED + rank)
    x = torch.empty(n_local, dtype=torch.float32, device=device).normal_(0, 1, generator=gen)
    y = torch.empty_like(x)

    def step():
        scan(x, out=y)
    for _ in range(warmup):
        step()
    barrier()
    scan.check_status()
    ms = time_steps(torch, step, steps, None, barrier)
    scan.check_status()
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # one GPU: the ring scan (one kernel); several: the shard total, then the ring scan seeded with the carry
    kernels_per_step = 1 if world == 1 else 2
    moved = 8 if world == 1 else 12
    e2e = None
    if with_e2e:
        host_in = torch.empty(n_local, dtype=torch.float32, pin_memory=True)
        host_in.copy_(x)
        host_out = torch.empty(n_local, dtype=torch.float32, pin_memory=True)
        e2e_steps = 3
        host_scan = parallel.HostScan(1 << 26, 'add') if world == 1 else None
        if host_scan is not None:
            host_scan(host_in, host_out)          # warm-up: streams, events, first launches
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            if host_scan is not None:
                # one GPU: chunks of the line stream through the device, both link directions busy at once
                host_scan(host_in, host_out)
            else:
                x.copy_(host_in, non_blocking=True)
                scan(x, out=y)
                host_out.copy_(y, non_blocking=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        e2e = {'value': n_local * world * e2e_steps / dt, 'unit': 'elements/s', 'h2d_bytes_per_step': n_local * 4 * world,
               'd2h_bytes_per_step': n_local * 4 * world, 'steps': e2e_steps, 'ms_per_step': dt / e2e_steps * 1e3,
               'api': 'parallel.HostScan (chunk-pipelined) from/to pinned host tensors' if world == 1 else
               'parallel.ShardedScan from/to pinned host tensors'}
    del x, y
    peak, _ = measured_peak()
    per_step = ms / steps
    achieved = 8.0 * n_local / (per_step * 1e-3) / 1e9
    return {'elements': n_local * world, 'elements_local': n_local, 'ms_per_step': per_step,
            'value': n_local * world / (per_step * 1e-3), 'kernels_per_step': kernels_per_step,
            'bytes_per_element_algorithmic': 8, 'bytes_per_element_moved': moved,
            'achieved_gbs_per_gpu': achieved, 'frac': achieved / peak,
            'frac_of_moved_bytes': achieved * moved / 8.0 / peak,
            'exchange': ('none (one GPU: single-pass ring scan)' if world == 1 else
                         'peer memory: totals stored into every rank\'s buffer by the reduction kernel, read by the '
                         'scan kernel (8 B per rank, no collective call)' if scan.exchange == 'peer' else
                         'all_gather of 8 B per rank between the two kernels'),
            'e2e': e2e}


def link_floor(torch, dist, world, device, nbytes_in, nbytes_out, barrier):
    """Bare pinned-memory copies of one step's bytes, host to device and device to host at the same time on two
    streams, all ranks at once: what the host side (links, host memory) allows the end-to-end leg."""
    hin = torch.empty(nbytes_in, dtype=torch.uint8, pin_memory=True)
    hout = torch.empty(nbytes_out, dtype=torch.uint8, pin_memory=True)
    din = torch.empty(nbytes_in, dtype=torch.uint8, device=device)
    dout = torch.empty(nbytes_out, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)
    best = None
    for _ in range(3):
        barrier()
        t0 = time.perf_counter()
        with torch.cuda.stream(s1):
            din.copy_(hin, non_blocking=True)
        with torch.cuda.stream(s2):
            hout.copy_(dout, non_blocking=True)
        s1.synchronize()
        s2.synchronize()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        best = dt if best is None else min(best, dt)
    return best * 1e3


def main():
    global C4_ROWS, C4_COLS, C5_TOTAL
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200')
    ap.add_argument('--workload', default='c4')
    ap.add_argument('--math', default='tolerance', choices=['tolerance', 'exact'],
                    help='math lowering of the generated kernels')
    ap.add_argument('--exchange', default='auto', choices=['auto', 'peer', 'collective'],
                    help='how the shards of c5 exchange their totals')
    ap.add_argument('--c4-rows', type=int, default=C4_ROWS, help='rows of the c4 tensor (profiling small cases)')
    ap.add_argument('--c4-cols', type=int, default=C4_COLS, help='columns of the c4 tensor (profiling small cases)')
    ap.add_argument('--c5-n', type=int, default=C5_TOTAL, help='elements of the c5 tensor (profiling small cases)')
    ap.add_argument('--no-cpu', action='store_true', help='skip the CPU baseline leg')
    ap.add_argument('--no-e2e', action='store_true', help='skip the end-to-end leg')
    ap.add_argument('--no-secondary', action='store_true', help='skip the exact-math and c5 legs after c4')
    args = ap.parse_args()
    if args.warmup < 3 and args.impl != 'reference':
        args.warmup = 3
    workload = args.workload
    C4_ROWS, C4_COLS, C5_TOTAL = args.c4_rows, args.c4_cols, args.c5_n
    if args.impl == 'reference':
        return run_reference_arm(args, workload)

    import torch
    import torch.distributed as dist
    rank, world, local = dist_env()
    if world != args.gpus:
        # plain `python bench.py --gpus N` with N > 1: launch one process per GPU
        if world == 1 and args.gpus > 1:
            cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', str(args.gpus),
                   '--master-addr', '127.0.0.1', '--master-port', str(29500 + os.getpid() % 1000), os.path.abspath(__file__)
                   ] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit('WORLD_SIZE does not match --gpus')
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    numa = bind_near_gpu(local)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)

    import opveclib_b200 as ovl
    from opveclib_b200 import runtime, parallel
    ovl.set_math_mode(args.math)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream_ptr = torch.cuda.current_stream().cuda_stream
    flush = None
    e2e = None
    steady = None
    same_size_copy_ms = None
    exact_math = None
    secondary = {}
    sampler = ClockSampler(local)
    if workload == 'c5':
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        c5 = run_c5(torch, dist, parallel, args, rank, world, device, barrier, args.steps, args.warmup, not args.no_e2e)
        clocks = sampler.stop() if rank == 0 else None
        elements_local, bytes_per_elem = c5['elements_local'], 8
        elapsed_ms = c5['ms_per_step'] * args.steps
        kernels_per_step = c5['kernels_per_step']
        e2e = c5.pop('e2e')
        secondary['c5_detail'] = c5
    else:
        if workload != 'c4' and world > 1:
            raise SystemExit('only c4 and c5 shard over several GPUs')
        rows_local = C4_ROWS // world if workload == 'c4' else None
        outs, elements_local, bytes_per_elem = build_graph(workload, rows_local=rows_local)
        prog, dag = runtime.compile_outputs(outs)
        ins = make_device_inputs(torch, workload, dag.input_types, device, SEED + rank)
        out_bufs = [torch.empty(prog.plans[o].out_types[k].shape, dtype=prog.plans[o].out_types[k].dtype.as_torch(),
                                device=device) for o, k in prog.dag.outputs]
        small = sum(t.size * t.dtype.itemsize for t in dag.input_types) <= 126 * 10 ** 6     # inputs that fit in L2
        if small:
            flush = torch.empty(192 << 20, dtype=torch.uint8, device=device)

        # the whole step is recorded once into a CUDA graph and replayed: several of the workloads run for a few
        # microseconds per kernel, less than it takes the host to enqueue them one by one
        graph = prog.capture(ins, local, out_bufs)

        def step():
            graph.replay()
        kernels_per_step = sum(len(p._passes(p.last_variant, local)) for p in prog.plans)

        for _ in range(args.warmup):
            step()
        barrier()
        prog.check_status(local, stream_ptr)
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        elapsed_ms = time_steps(torch, step, args.steps, flush, barrier)
        if flush is not None:
            # launch-bound sizes: also the steady state of back-to-back launches (inputs stay in L2 - reported
            # apart, never as the headline)
            reps = max(50, args.steps)
            ms = time_steps(torch, step, reps, None, barrier)
            steady = {'ms_per_step': ms / reps, 'steps': reps,
                      'note': 'back-to-back launches without the L2 flush: inputs are L2-resident'}
        clocks = sampler.stop() if rank == 0 else None
        prog.check_status(local, stream_ptr)
        # a plain streaming kernel (torch: dst = 2 * src) that moves the same number of bytes, timed the same way:
        # what the measured peak (a 2 GiB copy) becomes at this problem's size, where launch and ramp-up are a
        # visible share of the time
        copy_bytes = elements_local * bytes_per_elem // 2
        if world == 1 and copy_bytes <= (2 << 30):
            # (an element-wise kernel, not a memcpy node: inside a CUDA graph those may run on a copy engine)
            src = torch.empty(copy_bytes // 4, dtype=torch.float32, device=device).fill_(1)
            dst = torch.empty_like(src)
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                torch.mul(src, 2.0, out=dst)
            side.synchronize()
            copy_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(copy_graph, stream=side):
                torch.mul(src, 2.0, out=dst)
            for _ in range(3):
                copy_graph.replay()
            same_size_copy_ms = time_steps(torch, copy_graph.replay, args.steps, flush, barrier) / args.steps
            del src, dst
        if workload == 'c4' and args.math != 'exact' and not args.no_secondary:
            # the same graph with CUDA's libm and IEEE division
            xprog, _ = runtime.compile_outputs(outs, math='exact')
            xgraph = xprog.capture(ins, local, out_bufs)
            for _ in range(3):
                xgraph.replay()
            xsteps = max(3, min(args.steps, 5))
            xms = time_steps(torch, xgraph.replay, xsteps, None, barrier)
            tx = torch.tensor([xms], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(tx, op=dist.ReduceOp.MAX)
            exact_math = {'ms_per_step': float(tx.item()) / xsteps, 'steps': xsteps,
                          'note': "math='exact': CUDA libm and IEEE division, results within 1-2 ulp of the C++ operator"}
            del xgraph
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    total_elements = elements_local * world
    value = total_elements * args.steps / (elapsed_ms * 1e-3)

    # ---- end to end through the public API: pinned host arrays in, pinned host arrays out
    if not args.no_e2e and workload != 'c5':
        host_in = [torch.empty(tuple(tt.shape), dtype=tt.dtype.as_torch(), pin_memory=True) for tt in dag.input_types]
        for h, d in zip(host_in, ins):
            h.copy_(d)
        host_out = [torch.empty(tuple(b.shape), dtype=b.dtype, pin_memory=True) for b in out_bufs]
        np_in = [h.numpy() for h in host_in]
        np_out = [h.numpy() for h in host_out]
        graph_h = rebuild_with_inputs(workload, np_in, rows_local if workload == 'c4' else None)
        e2e_steps = max(3, min(args.steps, 10))
        ovl.evaluate(graph_h, target_language='b200', out=np_out)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ovl.evaluate(graph_h, target_language='b200', out=np_out)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        bytes_in, bytes_out = int(sum(a.nbytes for a in np_in)), int(sum(a.nbytes for a in np_out))
        e2e = {'value': total_elements * e2e_steps / dt, 'unit': 'elements/s',
               'h2d_bytes_per_step': bytes_in * world, 'd2h_bytes_per_step': bytes_out * world, 'steps': e2e_steps,
               'ms_per_step': dt / e2e_steps * 1e3,
               'api': "ovl.evaluate(outputs, target_language='b200', out=pinned) - rows streamed in slabs when the graph is row-local"}
        del host_in, host_out, np_in, np_out
        # what bare copies of the same bytes take, all ranks at once (no kernels, no slabs)
        e2e['link_floor_ms'] = link_floor(torch, dist, world, device, bytes_in, bytes_out, barrier)
        e2e['host'] = numa

    if workload == 'c4' and not args.no_secondary:
        # the one configuration whose shards communicate, on the same GPUs
        del ins, out_bufs, graph
        torch.cuda.empty_cache()
        c5_steps = max(3, min(args.steps, 10))
        secondary['c5'] = run_c5(torch, dist, parallel, args, rank, world, device, barrier, c5_steps, 3, False)
        secondary['c5'].pop('e2e', None)
        secondary['c5']['steps'] = c5_steps
        secondary['c5']['config'] = workload_config('c5', world)['workload']
        kernels_per_step_c5 = secondary['c5']['kernels_per_step']
    if rank == 0:
        peak, peak_kind = measured_peak()
        launch_ms = elapsed_ms / args.steps
        # the dominant kernel is the (single) fused kernel of a step; for c5 on several GPUs the reduction pass
        # belongs to the same step, so the per-step bytes are reported against the per-step time
        algo_bytes = bytes_per_elem * elements_local
        achieved = algo_bytes / (launch_ms * 1e-3) / 1e9
        config = workload_config(workload, world)
        config['math'] = args.math
        line = {
            'metric': 'fused-op elements/s', 'value': value, 'unit': 'elements/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': launch_ms, 'higher_is_better': True,
            'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f64' if workload == 'perf_accumulate' else 'f32',
            'data': 'synthetic', 'config': config,
            'effective_hbm_gbs': achieved * world, 'pct_of_8tbs_per_gpu': 100.0 * achieved / NOMINAL_HBM_GBS,
            'roofline': {'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak,
                         'peak_kind': peak_kind + ' HBM copy bandwidth', 'algorithmic_bytes_per_element': bytes_per_elem,
                         'traffic': profiled_traffic(workload, elements_local),
                         'same_size_copy_ms': same_size_copy_ms,
                         'frac_of_same_size_copy': (same_size_copy_ms / (elapsed_ms / args.steps)
                                                    if same_size_copy_ms else None)},
            'clocks': clocks, 'e2e': e2e, 'gpu_launches': kernels_per_step * args.steps,
        }
        if steady is not None:
            line['steady_state'] = steady
        if exact_math is not None:
            exact_math['frac'] = algo_bytes / (exact_math['ms_per_step'] * 1e-3) / 1e9 / peak
            line['exact_math'] = exact_math
        if secondary:
            line['secondary'] = secondary
        if world == 1 and not args.no_cpu:
            try:
                line['cpu_baseline'], _ = cpu_reference_run(workload, 7)
            except Exception as exc:   # the baseline is a report, never a reason to lose the GPU number
                line['cpu_baseline'] = {'error': '%s: %s' % (type(exc).__name__, exc)}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def rebuild_with_inputs(workload, np_inputs, rows_local):
    """The workload's operator graph over concrete host arrays (the e2e leg evaluates real data)."""
    from opveclib_b200.examples import workloads as cases
    ns = cases.namespace()
    if workload == 'c4':
        return [cases.chain16(ns, np_inputs[0])]
    if workload == 'light16':
        return [cases.chain16_light(ns, np_inputs[0])]
    if workload == 'c2_cumsum':
        return [ns.cumsum(np_inputs[0], axis=1)]
    if workload == 'c2_cumprod':
        return [ns.cumprod(np_inputs[0], axis=1)]
    if workload == 'c1':
        return [cases.c1_chain(ns, np_inputs[0])]
    if workload == 'c1_shift':
        return [cases.user_ops(ns).shift_cyclic(np_inputs[0])]
    if workload == 'matvec':
        return [cases.user_ops(ns).matvec(np_inputs[0], np_inputs[1])]
    if workload in ('colsum', 'colsum_narrow'):
        return [cases.user_ops(ns).colsum(np_inputs[0])]
    if workload == 'rowsum_short':
        return [cases.user_ops(ns).rowsum(np_inputs[0])]
    if workload == 'rownorm_short':
        return [cases.user_ops(ns).row_normalise(np_inputs[0])]
    if workload == 'scan_tiny':
        return [ns.cumsum(np_inputs[0], axis=1)]
    if workload == 'dot_long':
        mat, vec = sorted(np_inputs, key=lambda a: -a.ndim)
        return [cases.user_ops(ns).matvec(mat, vec)]
    if workload == 'rows_short':
        return [ns.cumsum(np_inputs[0], axis=1)]
    if workload == 'transpose':
        return [cases.user_ops(ns).transpose(np_inputs[0])]
    if workload == 'transpose_axpy':
        return [cases.user_ops(ns).transpose_axpy(np_inputs[0], np_inputs[1], alpha=0.5)]
    if workload in ('perf_accumulate', 'colscan', 'colscan_wide'):
        return [ns.cumsum(np_inputs[0], axis=0)]
    if workload == 'c3':
        op = ns.lstm(np_inputs[0], np_inputs[1], forget_bias=0.0)
        return [op[0], op[1]]
    if workload == 'c3_stdops':
        # (graph inputs come in the order the graph walk met them: tell the gates from the cell state by shape)
        gates, cell = sorted(np_inputs, key=lambda a: -a.shape[1])
        return cases.stdops_lstm(ns, gates, cell)
    if workload == 'c3_grad':
        op = ns.lstm_grad(np_inputs[0], np_inputs[1], np_inputs[2], np_inputs[3], forget_bias=0.0)
        return [op[0], op[1]]
    if workload.startswith('op_'):
        u, x = cases.user_ops(ns), np_inputs[0]
        single = {'op_tanh': lambda: u.ew_tanh(x), 'op_exp': lambda: u.ew_exp(x), 'op_log1p': lambda: ns.log1p(x),
                  'op_expm1': lambda: ns.expm1(x), 'op_mulc': lambda: u.ew_mulc(x, c=0.5), 'op_add': lambda: u.ew_add(x, x),
                  'op_where': lambda: u.where_greater(x, x)}
        return [single[workload]()]
    raise ValueError(workload)


if __name__ == '__main__':
    sys.exit(main())
