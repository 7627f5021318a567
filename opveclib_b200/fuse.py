"""Operator fusion: merge producer/consumer operators of an operator graph into single kernels.

Legality is the reference's rule (opveclib/operator.py:1150-1300, documentation/programming.rst:451-465): a
producer output feeding a consumer input can be merged when both operators have the same workgroup shape and
the consumer reads the tensor at exactly the index expression at which the producer's worker wrote it, so the
value can be handed over in a worker-local variable instead of through memory.  Unlike the reference, a
producer may write the tensor from several exclusive branches (``if_/elif_/else_`` each assigning the output,
which the reference refuses at operator.py:1217-1222) as long as every write uses the same index, and operators
containing ``elif_`` fuse like any other (the reference loses their workgroup shape, expression.py:420-435).
Fusion never changes arithmetic: statements keep their order and their types.

The merged body is the producer's statements followed by the consumer's (opveclib/operator.py:1453-1666):
internal tensors become variables, the consumer shares the producer's position, inputs that refer to the same
source are passed once, and outputs nobody outside the merged kernel needs disappear.
"""
import copy

from . import expr as E
from .access import analyze
from .dtypes import int64
from .kernel import KernelIR, iter_nodes
from .local import logger
from .opgraph import InputRef, OpDAG

_merged_registry = {}


def _raw(cls, **fields):
    node = cls.__new__(cls)
    node.args = []
    node.attr = {}
    for k, v in fields.items():
        setattr(node, k, v)
    return node


def _raw_tensor(cls, tensor_type, **attr):
    node = _raw(cls, tensor_type=tensor_type, dtype=tensor_type.dtype, shape=tensor_type.shape,
                size=tensor_type.size, rank=tensor_type.rank)
    node.attr = dict(attr)
    return node


def _struct_key(node, cache):
    """Structural identity of an index expression (used when no affine form exists)."""
    k = cache.get(id(node))
    if k is not None:
        return k
    if node.kind == 'const':
        k = ('c', node.dtype.code, node.attr['value'])
    elif node.kind == 'cast':
        k = ('cast', node.dtype.code, _struct_key(node.args[0], cache))
    elif node.kind == 'binary':
        k = ('b', node.attr['fn'], node.dtype.code, _struct_key(node.args[0], cache),
             _struct_key(node.args[1], cache))
    elif node.kind == 'unary':
        k = ('u', node.attr['fn'], node.dtype.code, _struct_key(node.args[0], cache))
    elif node.kind == 'read' and node.args[0].kind == 'position':
        k = ('p', _struct_key(node.args[1], cache))
    else:
        k = ('opaque', id(node))
    cache[id(node)] = k
    return k


def _index_key(access, info, cache):
    if access.form is not None:
        return ('affine',) + access.form.key()
    return ('struct', _struct_key(access.node.args[1], cache))


class _Group(object):
    """A (possibly already merged) kernel of the working graph."""

    def __init__(self, kernel, refs):
        self.kernel = kernel
        self.refs = refs            # list of ('L', leaf) / ('G', group, out_index)
        self._info = None

    @property
    def info(self):
        if self._info is None:
            self._info = analyze(self.kernel)
        return self._info


def _edge_mergeable(g, h, out_index, in_indices):
    """Can output ``out_index`` of group g be handed to inputs ``in_indices`` of group h in a variable?"""
    out_node = g.kernel.outputs[out_index]
    cache = {}
    wkeys = set()
    for acc in g.info.accesses:
        if acc.is_write and acc.tensor is out_node:
            if acc.loop_depth > 0:
                return False
            wkeys.add(_index_key(acc, g.info, cache))
    if len(wkeys) != 1:
        return False
    wkey = next(iter(wkeys))
    if wkey[0] == 'struct' and 'opaque' in repr(wkey):
        return False
    in_nodes = [h.kernel.inputs[i] for i in in_indices]
    for acc in h.info.accesses:
        if not acc.is_write and any(acc.tensor is n for n in in_nodes):
            if _index_key(acc, h.info, cache) != wkey:
                return False
    return True


def _clone_block(block, mapping, hooks, out_block):
    for node in block.nodes:
        repl = hooks(node, mapping, out_block)
        if repl is False:
            continue
        new = copy.copy(node)
        new.attr = dict(node.attr)
        new.args = [mapping[id(a)] for a in node.args]
        mapping[id(node)] = new
        if isinstance(node, E.ForRange):
            new.body = E.Block()
            _clone_block(node.body, mapping, hooks, new.body)
        elif isinstance(node, E.IfChain):
            new.conds = [None if c is None else mapping[id(c)] for c in node.conds]
            new.blocks = []
            for b in node.blocks:
                nb = E.Block()
                _clone_block(b, mapping, hooks, nb)
                new.blocks.append(nb)
        out_block.nodes.append(new)


def eliminate_dead_code(kernel):
    """Drop value nodes nothing uses and assignments to variables nothing reads."""
    nodes = list(iter_nodes(kernel.body))
    live = set()
    work = []

    def mark(n):
        if id(n) not in live:
            live.add(id(n))
            work.append(n)

    for n in nodes:
        if n.kind in ('assign_tensor', 'for', 'if', 'input', 'output', 'position'):
            mark(n)
    changed = True
    while changed:
        while work:
            n = work.pop()
            for a in n.args:
                mark(a)
            if isinstance(n, E.IfChain):
                for c in n.conds:
                    if c is not None:
                        mark(c)
        changed = False
        for n in nodes:
            if n.kind == 'assign_var' and id(n) not in live and id(n.args[0]) in live:
                mark(n)
                changed = True

    def prune(block):
        kept = []
        for n in block.nodes:
            if id(n) not in live:
                continue
            if isinstance(n, E.ForRange):
                prune(n.body)
            elif isinstance(n, E.IfChain):
                for b in n.blocks:
                    prune(b)
            kept.append(n)
        block.nodes = kept

    prune(kernel.body)
    kernel._text = None
    return kernel


def _merge_pair(g, h, internal, live_g_outputs):
    """Build the merged kernel of producer group g and consumer group h.

    internal         {h input index: g output index} for the tensors handed over in variables
    live_g_outputs   g output indices something other than h still needs
    Returns (kernel, refs, g_out_map, h_out_map) where the maps give new output indices."""
    body = E.Block()
    mapping = {}

    # inputs, deduplicated by source
    new_inputs, new_refs, by_source = [], [], {}

    def input_for(ref, tensor_type):
        key = ('L', id(ref[1])) if ref[0] == 'L' else ('G', id(ref[1]), ref[2])
        if key not in by_source:
            node = _raw_tensor(E.InputTensor, tensor_type, io_index=len(new_inputs))
            by_source[key] = node
            new_inputs.append(node)
            new_refs.append(ref)
            body.nodes.append(node)
        return by_source[key]

    for node, ref in zip(g.kernel.inputs, g.refs):
        mapping[id(node)] = input_for(ref, node.tensor_type)
    for i, (node, ref) in enumerate(zip(h.kernel.inputs, h.refs)):
        if i not in internal:
            mapping[id(node)] = input_for(ref, node.tensor_type)

    new_outputs, g_out_map, h_out_map = [], {}, {}
    for k, node in enumerate(g.kernel.outputs):
        if k in live_g_outputs:
            new = _raw_tensor(E.OutputTensor, node.tensor_type, io_index=len(new_outputs))
            g_out_map[k] = len(new_outputs)
            new_outputs.append(new)
            body.nodes.append(new)
            mapping[id(node)] = new
    for k, node in enumerate(h.kernel.outputs):
        new = _raw_tensor(E.OutputTensor, node.tensor_type, io_index=len(new_outputs))
        h_out_map[k] = len(new_outputs)
        new_outputs.append(new)
        body.nodes.append(new)
        mapping[id(node)] = new

    position = copy.copy(g.kernel.position)
    position.attr = dict(g.kernel.position.attr)
    position.args = []
    body.nodes.append(position)
    mapping[id(g.kernel.position)] = position
    mapping[id(h.kernel.position)] = position

    # one variable per handed-over tensor
    var_of_output = {}
    for k in sorted(set(internal.values())):
        t = g.kernel.outputs[k].tensor_type
        zero = _raw(E.ConstScalar, dtype=int64)
        zero.attr = {'value': 0}
        var = _raw(E.Variable, dtype=t.dtype)
        var.args = [zero]
        body.nodes.extend([zero, var])
        var_of_output[k] = var
    internal_out_nodes = {id(g.kernel.outputs[k]): k for k in var_of_output}
    internal_in_nodes = {id(h.kernel.inputs[i]): k for i, k in internal.items()}

    dead_out_nodes = set(id(n) for k, n in enumerate(g.kernel.outputs)
                         if k not in live_g_outputs and k not in var_of_output)

    def producer_hook(node, mapping, out_block):
        if node.kind in ('input', 'output', 'position'):
            return False
        if node.kind == 'assign_tensor' and id(node.args[0]) in dead_out_nodes:
            return False            # an output nothing consumes: the merged kernel does not produce it
        if node.kind == 'assign_tensor' and id(node.args[0]) in internal_out_nodes:
            k = internal_out_nodes[id(node.args[0])]
            assign = _raw(E.AssignVariable)
            assign.args = [var_of_output[k], mapping[id(node.args[2])]]
            if k in live_g_outputs:
                store = copy.copy(node)
                store.attr = dict(node.attr)
                store.args = [mapping[id(a)] for a in node.args]
                out_block.nodes.append(store)
            out_block.nodes.append(assign)
            return False
        return None

    def consumer_hook(node, mapping, out_block):
        if node.kind in ('input', 'output', 'position'):
            return False
        if node.kind == 'read' and id(node.args[0]) in internal_in_nodes:
            k = internal_in_nodes[id(node.args[0])]
            load = _raw(E.Cast, dtype=node.dtype)
            load.args = [var_of_output[k]]
            mapping[id(node)] = load
            out_block.nodes.append(load)
            return False
        return None

    _clone_block(g.kernel.body, mapping, producer_hook, body)
    _clone_block(h.kernel.body, mapping, consumer_hook, body)

    kernel = KernelIR(g.kernel.name + '+' + h.kernel.name, body, new_inputs, new_outputs, position)
    eliminate_dead_code(kernel)
    # inputs whose every read disappeared stay in the signature only if still referenced
    used = set()
    for n in iter_nodes(kernel.body):
        for a in n.args:
            used.add(id(a))
    keep = [i for i, n in enumerate(new_inputs) if id(n) in used]
    if len(keep) != len(new_inputs):
        kept_nodes = [new_inputs[i] for i in keep]
        dropped = set(id(n) for n in new_inputs) - set(id(n) for n in kept_nodes)
        kernel.body.nodes = [n for n in kernel.body.nodes if id(n) not in dropped]
        for idx, n in enumerate(kept_nodes):
            n.attr['io_index'] = idx
        kernel.inputs = kept_nodes
        new_refs = [new_refs[i] for i in keep]
        kernel._text = None
    return kernel, new_refs, g_out_map, h_out_map


def merge_op_dag(dag):
    """Fuse every legal producer/consumer pair of an operator graph, to a fixed point.  Returns a new OpDAG
    over the same leaf inputs and with the same outputs."""
    memo_key = dag.text()
    hit = _merged_registry.get(memo_key)
    if hit is not None:
        kernels, references, outputs = hit
        return OpDAG(kernels, references, dag.inputs, dag.input_types, outputs, [None] * len(kernels))

    groups = []
    for kernel, refs in zip(dag.kernels, dag.references):
        groups.append(_Group(kernel, None))
    for grp, refs in zip(groups, dag.references):
        grp.refs = [('L', ('leaf', r.dag_input_index)) if r.is_leaf else ('G', groups[r.op_index], r.op_output_index)
                    for r in refs]
    # leaves are identified by index; wrap in small objects so that id() is a stable key
    leaf_objs = {}
    for grp in groups:
        fixed = []
        for ref in grp.refs:
            if ref[0] == 'L':
                idx = ref[1][1]
                leaf_objs.setdefault(idx, ('leaf', idx))
                fixed.append(('L', leaf_objs[idx]))
            else:
                fixed.append(ref)
        grp.refs = fixed
    outputs = [(groups[o], k) for o, k in dag.outputs]

    def consumers_of(grp):
        res = []
        for other in groups:
            if other is grp:
                continue
            if any(r[0] == 'G' and r[1] is grp for r in other.refs):
                res.append(other)
        return res

    def reaches(src, dst, skip_direct_from):
        # is there a path src -> ... -> dst that does not start with the direct edge skip_direct_from -> dst
        seen, stack = set(), [c for c in consumers_of(src) if c is not dst]
        while stack:
            n = stack.pop()
            if n is dst:
                return True
            if id(n) in seen:
                continue
            seen.add(id(n))
            stack.extend(consumers_of(n))
        return False

    progress = True
    while progress:
        progress = False
        for h in list(groups):
            producers = []
            for r in h.refs:
                if r[0] == 'G' and not any(r[1] is p for p in producers):
                    producers.append(r[1])
            for g in producers:
                if g.kernel.workgroup_shape != h.kernel.workgroup_shape:
                    logger.info('Non-matching workgroup shapes: ' + g.kernel.name + ' -> ' + h.kernel.name)
                    continue
                internal, ok = {}, True
                by_out = {}
                for i, r in enumerate(h.refs):
                    if r[0] == 'G' and r[1] is g:
                        by_out.setdefault(r[2], []).append(i)
                for k, idxs in by_out.items():
                    if g.kernel.outputs[k].tensor_type != h.kernel.inputs[idxs[0]].tensor_type or \
                            not _edge_mergeable(g, h, k, idxs):
                        ok = False
                        break
                    for i in idxs:
                        internal[i] = k
                if not ok:
                    logger.info('Access patterns do not match: ' + g.kernel.name + ' -> ' + h.kernel.name)
                    continue
                if reaches(g, h, g):
                    continue
                live = set()
                for other in groups:
                    if other is h or other is g:
                        continue
                    for r in other.refs:
                        if r[0] == 'G' and r[1] is g:
                            live.add(r[2])
                for og, ok_ in outputs:
                    if og is g:
                        live.add(ok_)
                kernel, refs, g_map, h_map = _merge_pair(g, h, internal, live)
                merged = _Group(kernel, refs)
                logger.info('Merged ' + g.kernel.name + ' into ' + h.kernel.name)
                for other in groups:
                    if other is g or other is h:
                        continue
                    new_refs = []
                    for r in other.refs:
                        if r[0] == 'G' and r[1] is g:
                            new_refs.append(('G', merged, g_map[r[2]]))
                        elif r[0] == 'G' and r[1] is h:
                            new_refs.append(('G', merged, h_map[r[2]]))
                        else:
                            new_refs.append(r)
                    other.refs = new_refs
                outputs = [(merged, g_map[k]) if og is g else ((merged, h_map[k]) if og is h else (og, k))
                           for og, k in outputs]
                groups = [x for x in groups if x is not g and x is not h] + [merged]
                progress = True
                break
            if progress:
                break

    # topological order
    order, placed = [], set()
    remaining = list(groups)
    while remaining:
        for grp in remaining:
            if all(r[0] == 'L' or id(r[1]) in placed for r in grp.refs):
                order.append(grp)
                placed.add(id(grp))
                remaining.remove(grp)
                break
        else:
            raise RuntimeError('operator graph has a cycle after merging')
    index_of = {id(grp): i for i, grp in enumerate(order)}
    kernels = [grp.kernel for grp in order]
    references = []
    for grp in order:
        refs = []
        for r in grp.refs:
            if r[0] == 'L':
                refs.append(InputRef(True, dag_input_index=r[1][1]))
            else:
                refs.append(InputRef(False, op_index=index_of[id(r[1])], op_output_index=r[2]))
        references.append(refs)
    out = [(index_of[id(og)], k) for og, k in outputs]
    _merged_registry[memo_key] = (kernels, references, out)
    return OpDAG(kernels, references, dag.inputs, dag.input_types, out, [None] * len(kernels))
