"""A traced operator body (:class:`KernelIR`), its canonical serialisation and structural utilities.

KernelIR plays the role of the reference's ``ExpressionDAG`` message (opveclib/language.proto:394-404): the
ordered expression list of one parallel-for operator together with its workgroup shape and io signature.  The
canonical text produced by :func:`serialize` is what kernel caches are keyed on, as the reference keys on
the serialised protobuf (opveclib/operator.py:357-358).
"""
import hashlib
import json

from . import expr as E
from .dtypes import TensorType


class KernelIR(object):
    """One operator: inputs, outputs, workgroup shape and the structured body."""

    def __init__(self, name, body, inputs, outputs, position):
        self.name = name
        self.body = body              # E.Block
        self.inputs = inputs          # list of InputTensor nodes, ordered by io_index
        self.outputs = outputs        # list of OutputTensor nodes, ordered by io_index
        self.position = position      # PositionTensor node
        self._text = None

    @property
    def workgroup_shape(self):
        return list(self.position.workgroup_shape)

    @property
    def num_workers(self):
        n = 1
        for d in self.position.workgroup_shape:
            n *= d
        return n

    @property
    def input_types(self):
        return [n.tensor_type for n in self.inputs]

    @property
    def output_types(self):
        return [n.tensor_type for n in self.outputs]

    def text(self):
        if self._text is None:
            self._text = serialize(self)
        return self._text

    def digest(self):
        return hashlib.sha224(self.text().encode('utf-8')).hexdigest()


def iter_nodes(block):
    """All nodes of a block in program order, descending into loop and branch bodies."""
    for node in block.nodes:
        yield node
        if isinstance(node, E.ForRange):
            for sub in iter_nodes(node.body):
                yield sub
        elif isinstance(node, E.IfChain):
            for b in node.blocks:
                for sub in iter_nodes(b):
                    yield sub


def _ser_block(block, ids, out):
    for node in block.nodes:
        ids[id(node)] = len(ids)
        rec = [node.kind]
        if isinstance(node, E.Scalar):
            rec.append(node.dtype.code)
        if isinstance(node, E.TensorExpr):
            rec.append([node.dtype.code] + list(node.shape))
        if node.attr:
            rec.append({k: node.attr[k] for k in sorted(node.attr)})
        rec.append([ids[id(a)] for a in node.args])
        if isinstance(node, E.ForRange):
            sub = []
            _ser_block(node.body, ids, sub)
            rec.append(sub)
        elif isinstance(node, E.IfChain):
            branches = []
            for cond, b in zip(node.conds, node.blocks):
                sub = []
                _ser_block(b, ids, sub)
                branches.append([None if cond is None else ids[id(cond)], sub])
            rec.append(branches)
        out.append(rec)


def serialize(kernel):
    """Canonical JSON text of a kernel: node kinds, dtypes, attributes and operand numbers in program order.
    Two kernels have equal text iff they are structurally identical (names excluded)."""
    ids = {}
    body = []
    _ser_block(kernel.body, ids, body)
    return json.dumps({'workgroup': kernel.workgroup_shape, 'body': body}, separators=(',', ':'))


def finish_trace(builder, name, returned):
    """Turn a finished TraceBuilder into a KernelIR, renumbering outputs in return order
    (opveclib/operator.py:447-477)."""
    if returned is None:
        raise ValueError('No outputs returned from op function')
    if isinstance(returned, (list, tuple)):
        outs = list(returned)
    else:
        outs = [returned]
    if len(outs) != len(builder.outputs):
        raise ValueError('Defined ' + str(len(builder.outputs)) + ' outputs, but returned ' + str(len(outs)) +
                         '. Number of defined outputs must equal number of returned outputs.')
    seen = set()
    for index, node in enumerate(outs):
        if type(node) is not E.OutputTensor:
            raise TypeError('User functions must only return outputs. Instead got:\n' + str(node))
        if id(node) in seen:
            raise ValueError('The same output was returned more than once.')
        seen.add(id(node))
        node.attr['io_index'] = index
    if builder.position is None:
        raise ValueError('Workgroup shape must be defined with "position_in" function.')
    if len(builder.stack) != 1:
        raise SyntaxError('Unbalanced control flow blocks')
    return KernelIR(name, builder.root, list(builder.inputs), outs, builder.position)


def trace_function(fn, input_types, constants, name):
    """Trace ``fn(*inputs, **constants)`` into a KernelIR."""
    with E.tracing() as builder:
        input_exprs = [E.input(TensorType.like(t)) for t in input_types]
        returned = fn(*input_exprs, **constants)
        return finish_trace(builder, name, returned)
