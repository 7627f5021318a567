"""Row-streamed evaluation of host-resident operator graphs.

When the inputs of ``evaluate`` live in host memory, a whole-tensor run is copy in, compute, copy out, one
after the other - and PCIe, not the GPU, sets the time.  If every kernel of the graph treats the leading axis as
a batch axis (each worker touches only row ``position[0]`` of every tensor), the graph can be evaluated slab by
slab: while slab i is computed, slab i+1 travels to the device and slab i-1 travels back, so both directions of
the link are busy at once.  The slab-shaped graph is obtained by tracing the same operators again for the
smaller input shape (operators are shape-specialised at trace time, as in the reference,
opveclib/operator.py:410-445).

Row locality is proven from the affine index forms (access.py): an access qualifies when its offset is
``row_stride * position[0] + r`` with ``0 <= r < row_stride`` for a tensor whose leading extent is the
workgroup's, or when it does not depend on ``position[0]`` at all and the tensor is small (replicated to every
slab).  Anything else - loops, unproven indices, a tensor with another leading extent - and the graph is
evaluated in one piece as usual.

The first and the last slab travel alone (nothing to overlap with), so slabs should be small against the whole.
A graph with few rows is cut finer when it is *element-local*: all tensors have one shape and every worker
touches exactly the element at its own position.  Such a graph does not care how the elements are arranged, so
the tensors are viewed as ``[rows * k, columns / k, ...]`` (same memory) and streamed in slabs of those rows.
"""
import numpy as np

from .access import analyze
from .kernel import iter_nodes
from .opgraph import GradientPlaceholder, Operator, OperatorOutput, _resolve_output

MIN_BYTES = 32 << 20          # below this much leaf data one piece is as fast
MAX_SLABS = 8                 # row-local graphs
FINE_SLABS = 32               # element-local graphs
BUFFERS = 3                   # device-side slab buffers per tensor
_plans = {}


def _row_local(kernel, rows):
    """Every access of the kernel stays in row position[0]; returns False when that cannot be proven."""
    shape = kernel.workgroup_shape
    if len(shape) < 1 or shape[0] != rows:
        return False
    if any(n.kind in ('for', 'local') for n in iter_nodes(kernel.body)):
        return False
    info = analyze(kernel)
    p0 = ('p', 0)
    for acc in info.accesses:
        f = acc.form
        t = acc.tensor
        if f is None or f.mod is not None or t.kind not in ('input', 'output'):
            return False
        if not t.shape or t.shape[0] != rows:
            return False
        stride = t.size // rows
        if f.coef(p0) != stride:
            return False
        rest_lo = f.const + sum(min(c * info.ranges[s][0], c * info.ranges[s][1]) for s, c in f.coefs.items() if s != p0)
        rest_hi = f.const + sum(max(c * info.ranges[s][0], c * info.ranges[s][1]) for s, c in f.coefs.items() if s != p0)
        if rest_lo < 0 or rest_hi >= stride:
            return False
    # position[0] may not be used for anything but those indices (e.g. as a value)
    for n in iter_nodes(kernel.body):
        if n.kind == 'read' and n.args[0].kind == 'position':
            pass
    return not _position_value_escapes(kernel, info)


def _element_local(kernel, shape):
    """Every access of the kernel is the element at the worker's own position of a tensor of ``shape`` (the
    workgroup's shape), and the position is used for nothing else."""
    if list(kernel.workgroup_shape) != list(shape):
        return False
    if any(n.kind in ('for', 'local') for n in iter_nodes(kernel.body)):
        return False
    info = analyze(kernel)
    strides = [1]
    for d in range(len(shape) - 1, 0, -1):
        strides.append(strides[-1] * shape[d])
    strides.reverse()
    want = {('p', d): st for d, st in enumerate(strides) if shape[d] > 1}
    for acc in info.accesses:
        f, t = acc.form, acc.tensor
        if f is None or f.mod is not None or t.kind not in ('input', 'output') or list(t.shape) != list(shape):
            return False
        if f.const != 0 or {k: v for k, v in f.coefs.items()} != want:
            return False
    # no position entry may feed a value or a condition
    tainted = set()
    for n in iter_nodes(kernel.body):
        if n.kind == 'read' and n.args[0].kind == 'position':
            tainted.add(id(n))
        elif n.kind in ('cast', 'unary', 'binary') and any(id(a) in tainted for a in n.args):
            tainted.add(id(n))
        elif n.kind == 'assign_var' and id(n.args[1]) in tainted:
            return False
        elif n.kind == 'assign_tensor' and id(n.args[2]) in tainted:
            return False
        elif n.kind == 'if' and any(c is not None and id(c) in tainted for c in n.conds):
            return False
    return True


def _position_value_escapes(kernel, info):
    """True when position[0] feeds a stored value or a condition instead of only tensor indices."""
    tainted = set()
    for n in iter_nodes(kernel.body):
        if n.kind == 'read' and n.args[0].kind == 'position':
            f = info.form_of(n)
            if f is None or f.coef(('p', 0)) != 0:
                tainted.add(id(n))
        elif n.kind in ('cast', 'unary', 'binary') and any(id(a) in tainted for a in n.args):
            tainted.add(id(n))
        elif n.kind == 'assign_var' and id(n.args[1]) in tainted:
            return True
        elif n.kind == 'assign_tensor' and id(n.args[2]) in tainted:
            return True
        elif n.kind == 'if' and any(c is not None and id(c) in tainted for c in n.conds):
            return True
    return False


def _value_constants(kernel):
    """The constants that can reach a stored value, an assigned variable, a condition or a loop bound of the
    kernel other than through a tensor index, in program order.  Operators are specialised to their input shapes
    when traced, and a python number derived from a shape (``x[pos] / x.shape[0]``) becomes such a constant: a
    slab-shaped trace of that operator computes something else than the full-shaped one."""
    nodes = list(iter_nodes(kernel.body))
    reach = set()
    work = []
    for n in nodes:
        if n.kind == 'assign_tensor':
            work.append(n.args[2])
        elif n.kind == 'assign_var':
            work.append(n.args[1])
        elif n.kind == 'if':
            work.extend(c for c in n.conds if c is not None)
        elif n.kind == 'for':
            work.extend(n.args[1:])
        elif n.kind == 'variable':
            work.append(n.args[0])
    while work:
        n = work.pop()
        if id(n) in reach:
            continue
        reach.add(id(n))
        if n.kind == 'read':
            continue                      # (what it reads is data; its index is checked by the locality proofs)
        work.extend(a for a in n.args if getattr(a, 'is_scalar', False))
    return [(n.dtype.name, n.attr['value']) for n in nodes if n.kind == 'const' and id(n) in reach]


def _same_values(prog, slab_prog):
    """The slab-shaped program computes with the same constants as the full-shaped one."""
    if len(prog.dag.kernels) != len(slab_prog.dag.kernels):
        return False
    return all(_value_constants(a) == _value_constants(b) for a, b in zip(prog.dag.kernels, slab_prog.dag.kernels))


def _retrace(outputs, rows, slab_rows, trailing=None):
    """The same operator graph traced for slabs of ``slab_rows`` rows (with the trailing extents ``trailing``
    instead of the leaves' own when given).  Returns (slab outputs, leaf map: original leaf id -> placeholder),
    or None when an operator cannot be traced again."""
    memo, leaves = {}, {}

    def leaf(x):
        if id(x) not in leaves:
            shape = list(x.shape)
            if not shape or shape[0] != rows:
                return None
            rest = shape[1:] if trailing is None else list(trailing)
            leaves[id(x)] = (x, GradientPlaceholder([slab_rows] + rest, x.dtype))
        return leaves[id(x)][1]

    def build(op):
        if id(op) in memo:
            return memo[id(op)]
        if op.generator is None:
            return None
        args = []
        for inp in op.inputs:
            if isinstance(inp, (Operator, OperatorOutput)):
                r = _resolve_output(inp)
                parent = build(r.parent)
                if parent is None:
                    return None
                args.append(parent[r.index])
            else:
                ph = leaf(inp)
                if ph is None:
                    return None
                args.append(ph)
        new = op.generator(*args, **op.constants)
        # gradient placeholders switch gradient tracing off; nothing else differs
        memo[id(op)] = new
        return new

    slab_outputs = []
    for o in outputs:
        r = _resolve_output(o)
        parent = build(r.parent)
        if parent is None:
            return None
        slab_outputs.append(parent[r.index])
    return slab_outputs, leaves


def plan(output_list, dag, prog, opt_level):
    """A streaming plan for host inputs, or None.  Cached per graph structure."""
    from . import runtime
    key = (dag.text(), opt_level >= 3, prog.math)
    if key in _plans:
        return _plans[key]
    result = None
    try:
        rows = None
        ok = bool(dag.inputs) and opt_level >= 3
        for t in dag.input_types:
            if not t.shape or (rows is not None and t.shape[0] != rows):
                ok = False
            rows = t.shape[0] if t.shape else None
        total = sum(t.size * t.dtype.itemsize for t in dag.input_types)
        if ok and rows and total >= MIN_BYTES:
            result = _plan_element_local(output_list, dag, prog, opt_level, rows)
        if result is None and ok and rows and rows >= 2 and total >= MIN_BYTES:
            slabs = next((c for c in range(min(MAX_SLABS, rows), 1, -1) if rows % c == 0), None)
            if slabs and all(_row_local(k, rows) for k in prog.dag.kernels):
                out_ok = all(prog.plans[o].out_types[k].shape[0] == rows for o, k in prog.dag.outputs)
                traced = _retrace(output_list, rows, rows // slabs) if out_ok else None
                if traced is not None:
                    slab_outputs, leaves = traced
                    slab_prog, slab_dag = runtime.compile_outputs(slab_outputs, opt_level)
                    order = []
                    for ph in slab_dag.inputs:
                        orig = next(o for o, p in leaves.values() if p is ph)
                        order.append(next(i for i, x in enumerate(dag.inputs) if x is orig))
                    if _same_values(prog, slab_prog):
                        result = {'slabs': slabs, 'rows': rows, 'slab_rows': rows // slabs, 'prog': slab_prog,
                                  'leaf_order': order, 'view': None}
    except Exception:      # any doubt: evaluate in one piece
        result = None
    _plans[key] = result
    return result


def _plan_element_local(output_list, dag, prog, opt_level, rows):
    """Plan for a graph all of whose tensors share one shape and whose workers touch only their own element:
    the tensors are viewed as [rows * k, columns / k, ...] and streamed in FINE_SLABS slabs or fewer."""
    from . import runtime
    shape = list(dag.input_types[0].shape)
    if len(shape) < 2 or any(list(t.shape) != shape for t in dag.input_types):
        return None
    if any(list(prog.plans[o].out_types[k].shape) != shape for o, k in prog.dag.outputs):
        return None
    if not all(_element_local(k, shape) for k in prog.dag.kernels):
        return None
    cols = shape[1]
    best = None
    for k in range(1, FINE_SLABS + 1):
        if cols % k == 0 and rows * k <= FINE_SLABS and (cols // k) % 4 == 0:
            best = k
    if best is None or rows * best < 2:
        return None
    view_rows, trailing = rows * best, [cols // best] + shape[2:]
    # one slab per viewed row
    traced = _retrace(output_list, rows, 1, trailing)
    if traced is None:
        return None
    slab_outputs, leaves = traced
    slab_prog, slab_dag = runtime.compile_outputs(slab_outputs, opt_level)
    if not _same_values(prog, slab_prog):
        return None
    order = []
    for ph in slab_dag.inputs:
        orig = next(o for o, p in leaves.values() if p is ph)
        order.append(next(i for i, x in enumerate(dag.inputs) if x is orig))
    return {'slabs': view_rows, 'rows': view_rows, 'slab_rows': 1, 'prog': slab_prog, 'leaf_order': order,
            'view': [view_rows] + trailing}


def run(plan_, host_inputs, host_outputs, out_types, device):
    """Execute a streaming plan: ``host_inputs`` / ``host_outputs`` are numpy arrays (pinned memory makes the
    copies asynchronous), full-size; slabs rotate through three buffers on the device."""
    import torch
    prog = plan_['prog']
    slabs, sr = plan_['slabs'], plan_['slab_rows']
    dev = 'cuda:%d' % device
    ins_h = [torch.from_numpy(host_inputs[i]) for i in plan_['leaf_order']]
    outs_h = [torch.from_numpy(a) for a in host_outputs]
    if plan_.get('view') is not None:
        # element-local graph: same memory, more and shorter rows
        ins_h = [h.view(plan_['view']) for h in ins_h]
        outs_h = [h.view(plan_['view']) for h in outs_h]
    with torch.cuda.device(device):
        main = torch.cuda.current_stream()
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        for s in (s_in, s_run, s_out):
            s.wait_stream(main)
        # three slabs in flight: one travelling in, one being computed, one travelling out, whatever their order
        d_in = [[torch.empty((sr,) + tuple(h.shape[1:]), dtype=h.dtype, device=dev) for h in ins_h]
                for _ in range(BUFFERS)]
        d_out = [[torch.empty((sr,) + tuple(h.shape[1:]), dtype=h.dtype, device=dev) for h in outs_h]
                 for _ in range(BUFFERS)]
        loaded = [None] * BUFFERS
        computed = [None] * BUFFERS
        stored = [None] * BUFFERS
        for i in range(slabs):
            b = i % BUFFERS
            lo, hi = i * sr, (i + 1) * sr
            with torch.cuda.stream(s_in):
                if computed[b] is not None:
                    s_in.wait_event(computed[b])          # the slab that used this input buffer is done
                for d, h in zip(d_in[b], ins_h):
                    d.copy_(h[lo:hi], non_blocking=True)
                loaded[b] = torch.cuda.Event()
                loaded[b].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(loaded[b])
                if stored[b] is not None:
                    s_run.wait_event(stored[b])           # the result that sat in this output buffer has left
                prog.run(d_in[b], device, s_run.cuda_stream, None, d_out[b])
                computed[b] = torch.cuda.Event()
                computed[b].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[b])
                for d, h in zip(d_out[b], outs_h):
                    h[lo:hi].copy_(d, non_blocking=True)
                stored[b] = torch.cuda.Event()
                stored[b].record(s_out)
        for s in (s_in, s_run, s_out):
            main.wait_stream(s)
        main.synchronize()
        prog.check_status(device, main.cuda_stream)
    return host_outputs
