"""Recognition of loop idioms that have a cooperative kernel template.

The only idiom so far is the inclusive scan: one worker per line walks the line serially, combining a running
value with each element and storing it (``accumulate`` in opveclib/examples/test_accumulate.py:22-78, also the
zero-seeded form of opveclib/test/test_operator_merge.py:56-68).  Recognition is deliberately narrow - anything
that does not match exactly runs through the generic one-thread-per-worker kernel, which is always correct.
"""
from .access import analyze
from .kernel import iter_nodes

#: lines shorter than this stay on the generic kernel (a thread block per tile would mostly idle)
SCAN_MIN_AXIS = 1024


class ScanSpec(object):
    """``lines`` contiguous lines of ``n`` elements, inclusive scan with ``op`` ('add' or 'mul')."""

    def __init__(self, op, lines, n, dtype):
        self.op = op
        self.lines = lines
        self.n = n
        self.dtype = dtype


def _row_major_strides(shape):
    strides = [1]
    for d in range(len(shape) - 1, 0, -1):
        strides.append(strides[-1] * shape[d])
    strides.reverse()
    return strides


def match_scan(kernel, info=None):
    """ScanSpec if the kernel is exactly an inclusive scan along the contiguous axis of its only input into its
    only output, else None."""
    if len(kernel.inputs) != 1 or len(kernel.outputs) != 1:
        return None
    x, y = kernel.inputs[0], kernel.outputs[0]
    if x.tensor_type != y.tensor_type:
        return None
    top = kernel.body.nodes
    loops = [n for n in top if n.kind == 'for']
    if len(loops) != 1:
        return None
    loop = loops[0]
    all_nodes = list(iter_nodes(kernel.body))
    if any(n.kind in ('if', 'local') for n in all_nodes):
        return None
    if sum(1 for n in all_nodes if n.kind == 'for') != 1:
        return None

    info = info or analyze(kernel)
    var = loop.args[0]
    sym = info.loop_vars.get(id(var))
    if sym is None:
        return None
    step = info.form_of(loop.args[3])
    if step is None or not step.is_const() or step.const != 1:
        return None
    start, last = info.ranges[sym]
    if start not in (0, 1):
        return None
    n = last + 1

    # accesses: [pre-loop read, pre-loop write,] loop read, loop write
    accs = info.accesses
    loop_accs = [a for a in accs if a.loop_depth == 1]
    pre_accs = [a for a in accs if a.loop_depth == 0]
    if len(loop_accs) != 2 or loop_accs[0].is_write or not loop_accs[1].is_write:
        return None
    rd, wr = loop_accs
    if rd.tensor is not x or wr.tensor is not y or rd.form is None or wr.form is None or rd.form != wr.form:
        return None
    form = rd.form
    if form.mod is not None or form.const != 0 or form.coef(sym) != 1:
        return None
    shape = kernel.workgroup_shape
    lines = kernel.num_workers
    for d, s in enumerate(_row_major_strides(shape)):
        want = s * n if shape[d] > 1 else form.coef(('p', d))
        if form.coef(('p', d)) != want:
            return None
    if set(form.coefs) - set([sym] + [('p', d) for d in range(len(shape))]):
        return None
    if x.size != lines * n:
        return None

    # the running value
    assigns = [a for a in all_nodes if a.kind == 'assign_var']
    targets = set(id(a.args[0]) for a in assigns)
    if len(targets) != 1:
        return None
    acc = assigns[0].args[0]
    if acc.dtype != x.dtype:
        return None
    in_loop = set(id(nn) for nn in iter_nodes(loop.body))
    loop_assigns = [a for a in assigns if id(a) in in_loop]
    pre_assigns = [a for a in assigns if id(a) not in in_loop]
    if len(loop_assigns) != 1:
        return None
    upd = loop_assigns[0].args[1]
    if upd.kind != 'binary' or upd.attr['fn'] not in ('add', 'mul'):
        return None
    a, b = upd.args
    if not ((a is acc and b is rd.node) or (b is acc and a is rd.node)):
        return None
    if wr.node.args[2] is not acc:
        return None
    # statement order inside the loop: read, update, store
    order = [id(nn) for nn in loop.body.nodes]
    try:
        if not (order.index(id(rd.node)) < order.index(id(upd)) < order.index(id(loop_assigns[0])) <
                order.index(id(wr.node))):
            return None
    except ValueError:
        return None
    op = upd.attr['fn']

    init = acc.args[0].attr['value']
    if start == 1:
        # seeded with the first element: acc = x[line, 0]; y[line, 0] = acc
        if len(pre_accs) != 2 or pre_accs[0].is_write or not pre_accs[1].is_write or len(pre_assigns) != 1:
            return None
        prd, pwr = pre_accs
        if prd.tensor is not x or pwr.tensor is not y or prd.form is None or prd.form != pwr.form:
            return None
        expect = dict(form.coefs)
        expect.pop(sym, None)
        if prd.form.coefs != expect or prd.form.const != 0 or prd.form.mod is not None:
            return None
        if pre_assigns[0].args[1] is not prd.node or pwr.node.args[2] is not acc:
            return None
    else:
        if pre_accs or pre_assigns:
            return None
        identity = 0 if op == 'add' else 1
        if init != identity:
            return None
    # nothing else may observe the running value or the loop variable after the loop
    loop_at = [i for i, nn in enumerate(top) if nn is loop][0]
    after = top[loop_at + 1:]
    if any(nn.kind not in ('const', 'const_tensor') for nn in after):
        return None
    if x.dtype.name == 'float16':
        return None
    return ScanSpec(op, lines, n, x.dtype)
