"""Recognition of loop idioms that have a cooperative kernel template.

Two idioms: the inclusive scan - one worker per line walks the line serially, combining a running value with
each element and storing it (``accumulate`` in opveclib/examples/test_accumulate.py:22-78, also the zero-seeded
form of opveclib/test/test_operator_merge.py:56-68) - and the per-worker reduction loop - a worker folds a
computed term into one accumulator over a counted loop and uses the result afterwards (``dot`` in
opveclib/test/test_dot_product.py:18-34, the matrix-vector product of documentation/programming.rst:320-344).
Recognition is deliberately narrow - anything that does not match exactly runs through the generic
one-thread-per-worker kernel, which is always correct.
"""
from .access import analyze
from .kernel import iter_nodes

#: lines shorter than this stay on the generic kernel (a thread block per tile would mostly idle)
SCAN_MIN_AXIS = 1024


class ScanSpec(object):
    """Inclusive scan with ``op`` ('add' or 'mul') along the middle axis of a tensor seen as ``[outer, n, inner]``:
    ``lines = outer * inner`` lines of ``n`` elements.  ``inner == 1``: the lines are contiguous."""

    def __init__(self, op, lines, n, dtype, outer=None, inner=1):
        self.op = op
        self.lines = lines
        self.n = n
        self.dtype = dtype
        self.outer = lines if outer is None else outer
        self.inner = inner


#: scans along a non-contiguous axis shorter than this stay on the generic kernel (one thread per line already
#: reads whole row segments there; the cooperative version pays off when lines are long)
COLSCAN_MIN_AXIS = 256


def _row_major_strides(shape):
    strides = [1]
    for d in range(len(shape) - 1, 0, -1):
        strides.append(strides[-1] * shape[d])
    strides.reverse()
    return strides


def match_scan(kernel, info=None):
    """ScanSpec if the kernel is exactly an inclusive scan along one axis of its only input into its only output
    (one worker per line, workgroup = the tensor's shape without that axis), else None."""
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
    if form.mod is not None or form.const != 0 or form.coef(sym) < 1:
        return None
    shape = kernel.workgroup_shape
    lines = kernel.num_workers
    if set(form.coefs) - set([sym] + [('p', d) for d in range(len(shape))]):
        return None
    if x.size != lines * n:
        return None
    # which axis of the tensor is scanned: its extent is n and its row-major stride the loop variable's
    # coefficient; the workgroup's axes must then be the tensor's other axes, in order, with their strides
    tshape = list(x.shape)
    tstrides = _row_major_strides(tshape)
    geometry = None
    for axis in range(len(tshape)):
        if tshape[axis] != n or tstrides[axis] != form.coef(sym):
            continue
        others = [d for d in range(len(tshape)) if d != axis]
        if not others:
            ok = list(shape) == [1]
        else:
            ok = len(others) == len(shape) and all(
                shape[k] == tshape[d] and (tshape[d] == 1 or form.coef(('p', k)) == tstrides[d])
                for k, d in enumerate(others))
        if ok:
            outer = 1
            for d in range(axis):
                outer *= tshape[d]
            geometry = (outer, lines // outer)
            break
    if geometry is None:
        return None
    outer, inner = geometry

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
        # statement order in front of the loop: read, assign, store (a store in front of the assignment would
        # write the variable's initial value, not the first element)
        before = [id(nn) for nn in top]
        try:
            if not (before.index(id(prd.node)) < before.index(id(pre_assigns[0])) < before.index(id(pwr.node))):
                return None
        except ValueError:
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
    return ScanSpec(op, lines, n, x.dtype, outer, inner)


#: reduction loops shorter than this stay on the generic kernel
REDUCE_MIN_TRIPS = 128


class ReduceSpec(object):
    """A worker's counted loop ``acc = acc (op) term(position, i)`` for i in [0, n): ``loop`` is the loop node,
    ``acc`` the accumulator variable, ``update`` the assignment inside the loop, ``term`` the folded-in expression.
    For a nest of two loops (``for i: for j: acc += a[w, i, j]``) ``loop`` is the outer one, ``inner`` the inner one,
    ``n`` the product of the trip counts and ``n_inner`` the inner trip count: trip t of the flattened loop is
    i = t / n_inner, j = t % n_inner."""

    def __init__(self, op, n, loop, acc, update, term, inner=None, n_inner=None):
        self.op = op
        self.n = n
        self.loop = loop
        self.acc = acc
        self.update = update
        self.term = term
        self.inner = inner
        self.n_inner = n_inner

    @property
    def fastest_var(self):
        """The loop variable that changes from one trip to the next."""
        return (self.loop if self.inner is None else self.inner).args[0]


def _depends_on(node, targets, seen=None):
    seen = seen if seen is not None else set()
    if id(node) in seen:
        return False
    seen.add(id(node))
    if id(node) in targets:
        return True
    return any(_depends_on(a, targets, seen) for a in getattr(node, 'args', ()) if a is not None)


def match_reduce(kernel, info=None):
    """ReduceSpec if every worker of the kernel is: statements, ONE counted loop (start 0, step 1, constant trip
    count) whose only effect is folding a term into one accumulator with + or *, statements - else None.  The
    term may be any expression of the position, the loop variable and tensor reads; nothing inside the loop may
    write a tensor or observe the accumulator.  A nest of two such loops whose outer body holds nothing but value
    computations and the inner loop counts as one loop over the pairs (i, j) in row-major order."""
    top = kernel.body.nodes
    all_nodes = list(iter_nodes(kernel.body))
    if any(n.kind in ('if', 'local') for n in all_nodes):
        return None
    loops = [n for n in all_nodes if n.kind == 'for']
    if len(loops) not in (1, 2) or not any(x is loops[0] for x in top):
        return None
    loop = loops[0]
    info = info or analyze(kernel)

    def trips_from_zero(lp):
        sym = info.loop_vars.get(id(lp.args[0]))
        step = info.form_of(lp.args[3])
        if sym is None or step is None or not step.is_const() or step.const != 1:
            return None
        start, last = info.ranges[sym]
        return last + 1 if start == 0 else None

    var = loop.args[0]
    n = trips_from_zero(loop)
    if n is None:
        return None
    inner, n_inner = None, None
    if len(loops) == 2:
        inner = loops[1]
        # the outer body: the inner loop and, around it, nothing that has an effect
        if not any(x is inner for x in loop.body.nodes):
            return None
        if any(x.kind not in ('const', 'cast', 'variable', 'unary', 'binary', 'read', 'limit')
               for x in loop.body.nodes if x is not inner):
            return None
        n_inner = trips_from_zero(inner)
        if n_inner is None:
            return None
        n *= n_inner
    if n < REDUCE_MIN_TRIPS:
        return None
    assigns = [a for a in all_nodes if a.kind == 'assign_var']
    in_loop = list(iter_nodes(loop.body))
    in_loop_ids = set(id(x) for x in in_loop)
    if len(assigns) != 1 or id(assigns[0]) not in in_loop_ids:
        return None
    update = assigns[0]
    acc, value = update.args
    if acc.kind != 'variable' or not any(x is acc for x in top) or acc is var or acc.dtype.name == 'float16':
        return None
    if inner is not None and (acc is inner.args[0] or id(update) not in set(id(x) for x in inner.body.nodes)):
        return None
    if value.kind != 'binary' or value.attr['fn'] not in ('add', 'mul') or value.dtype != acc.dtype:
        return None
    a, b = value.args
    if a is acc and b is not acc:
        term = b
    elif b is acc and a is not acc:
        term = a
    else:
        return None
    if _depends_on(term, {id(acc), id(value)}):
        return None
    # inside the loop only the update may mention the accumulator; nothing may write a tensor
    for node in in_loop:
        if node.kind == 'assign_tensor':
            return None
        if node is value or node is update:
            continue
        if any(x is acc for x in getattr(node, 'args', ()) if x is not None):
            return None
    # before the loop the accumulator is only declared; after it the loop variable is dead
    at = [i for i, x in enumerate(top) if x is loop][0]
    for node in top[:at]:
        if node is not acc and any(x is acc for x in getattr(node, 'args', ()) if x is not None):
            return None
    if acc.args[0].kind != 'const':
        return None
    for node in top[at + 1:]:
        if any(x is var or (inner is not None and x is inner.args[0]) for x in getattr(node, 'args', ()) if x is not None):
            return None
    return ReduceSpec(value.attr['fn'], n, loop, acc, update, term, inner, n_inner)
