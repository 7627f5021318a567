"""Backward operator graphs from user-defined gradients.

Every operator may carry a gradient graph (``@gradient``): an operator graph over (operator inputs..., output
gradients...) producing one gradient per input (opveclib/operator.py:483-553).  The reference hands each
operator's gradient graph to TensorFlow, which chains them op by op (operator.py:84-123); here the chain rule is
applied on the operator graph itself: the gradient graphs of all operators on the path are inlined, in reverse
dependency order, into ONE operator graph over (forward leaves..., gradients of the requested outputs...).
Forward operators whose results a gradient needs are part of that graph (recomputed), so the fusion pass can
merge them with the gradient operators into the same kernels - the counterpart of the reference's merged
gradient graphs (operator.py:1701-1921), where ``gradient_sum`` and ``zeros`` helper operators accumulate
contributions (operator.py:1834-1855).
"""
from . import expr as E
from .opgraph import InputRef, OpDAG, GradientPlaceholder, operator


@operator()
def gradient_sum(a, b):
    """Sum of two gradient contributions to the same tensor."""
    out = E.output_like(a)
    pos = E.position_in(a.shape)
    out[pos] = a[pos] + b[pos]
    return out


@operator()
def zeros_like(x):
    """Zero gradient for an output nothing downstream depends on."""
    out = E.output_like(x)
    pos = E.position_in(x.shape)
    out[pos] = 0
    return out


class MissingGradient(Exception):
    pass


def compose_backward(dag):
    """Backward graph of an operator graph.

    Returns (OpDAG, has_grad): the graph's inputs are the forward leaves followed by one gradient per forward
    output; its outputs are the gradients of the leaves for which ``has_grad`` is True, in leaf order.  A leaf
    gets no gradient when no requested output depends on it or when an operator on the way has no gradient."""
    n_leaves = len(dag.input_types)
    out_types = [dag.kernels[o].output_types[k] for o, k in dag.outputs]
    leaf_types = list(dag.input_types) + out_types
    placeholders = [GradientPlaceholder(t.shape, t.dtype) for t in leaf_types]

    nodes = []   # [kernel, refs]
    for kernel, refs in zip(dag.kernels, dag.references):
        nodes.append([kernel, [InputRef(r.is_leaf, r.dag_input_index, r.op_index, r.op_output_index) for r in refs]])

    def type_of(ref):
        return leaf_types[ref.dag_input_index] if ref.is_leaf else nodes[ref.op_index][0].output_types[ref.op_output_index]

    def helper(gen, refs):
        types = [type_of(r) for r in refs]
        op = gen(*[GradientPlaceholder(t.shape, t.dtype) for t in types])
        nodes.append([op.kernel, list(refs)])
        return InputRef(False, op_index=len(nodes) - 1, op_output_index=0)

    def combine(refs):
        total = refs[0]
        for r in refs[1:]:
            total = helper(gradient_sum, [total, r])
        return total

    contributions = {}   # ('O', op, out) / ('L', leaf) -> [InputRef]
    for j, (o, k) in enumerate(dag.outputs):
        contributions.setdefault(('O', o, k), []).append(InputRef(True, dag_input_index=n_leaves + j))
    blocked = set()      # tensors whose gradient cannot be formed because an operator lacks a gradient

    for op in range(len(dag.kernels) - 1, -1, -1):
        kernel = dag.kernels[op]
        n_in, n_out = len(kernel.inputs), len(kernel.outputs)
        keys = [('O', op, k) for k in range(n_out)]
        if not any(key in contributions for key in keys):
            continue
        gd = dag.grad_dags[op]
        src_refs = nodes[op][1]
        if gd is None:
            for r in src_refs:
                blocked.add(('L', r.dag_input_index) if r.is_leaf else ('O', r.op_index, r.op_output_index))
            continue
        gout = []
        for k, key in enumerate(keys):
            srcs = contributions.get(key, [])
            if not srcs:
                gout.append(helper(zeros_like, [InputRef(False, op_index=op, op_output_index=k)]))
            else:
                gout.append(combine(srcs))
        base = len(nodes)
        for gk, grefs in zip(gd.kernels, gd.references):
            new_refs = []
            for r in grefs:
                if r.is_leaf:
                    i = r.dag_input_index
                    src = src_refs[i] if i < n_in else gout[i - n_in]
                    new_refs.append(InputRef(src.is_leaf, src.dag_input_index, src.op_index, src.op_output_index))
                else:
                    new_refs.append(InputRef(False, op_index=base + r.op_index, op_output_index=r.op_output_index))
            nodes.append([gk, new_refs])
        for i, (go, gko) in enumerate(gd.outputs):
            src = src_refs[i]
            key = ('L', src.dag_input_index) if src.is_leaf else ('O', src.op_index, src.op_output_index)
            contributions.setdefault(key, []).append(InputRef(False, op_index=base + go, op_output_index=gko))

    # a tensor downstream of a gradient-less operator poisons everything that only reaches outputs through it;
    # keep it simple and conservative: a blocked leaf gets no gradient at all
    outputs, has_grad = [], []
    for leaf in range(n_leaves):
        srcs = contributions.get(('L', leaf), [])
        if srcs and ('L', leaf) not in blocked:
            outputs.append(combine(srcs))
            has_grad.append(True)
        else:
            has_grad.append(False)

    # keep only what the requested gradients depend on, preserving order
    needed = set()
    stack = [r.op_index for r in outputs]
    while stack:
        i = stack.pop()
        if i in needed:
            continue
        needed.add(i)
        for r in nodes[i][1]:
            if not r.is_leaf:
                stack.append(r.op_index)
    order = sorted(needed)
    renum = {old: new for new, old in enumerate(order)}
    kernels, references = [], []
    for old in order:
        kernel, refs = nodes[old]
        kernels.append(kernel)
        references.append([InputRef(True, dag_input_index=r.dag_input_index) if r.is_leaf else
                           InputRef(False, op_index=renum[r.op_index], op_output_index=r.op_output_index) for r in refs])
    dag_outputs = [(renum[r.op_index], r.op_output_index) for r in outputs]
    bdag = OpDAG(kernels, references, placeholders, leaf_types, dag_outputs, [None] * len(kernels))
    return bdag, has_grad
