"""PyTorch bridge: operator graphs as differentiable torch functions.

Replaces the reference's TensorFlow bridge (``as_tensorflow`` / ``_dag_to_tf`` and the ``DynamicLib`` custom op,
opveclib/operator.py:2338-2412, opveclib/dynamiclibop.cc): leaf inputs are torch CUDA tensors, kernels run on
torch's current stream through the C-ABI launcher, outputs are torch tensors.  Gradients come from the
operators' own ``@gradient`` definitions, composed into one backward operator graph (autodiff.py) that is fused
and compiled like any other graph; ``torch.autograd`` only sees a single function.
"""
import numpy as np

from . import runtime
from .autodiff import compose_backward
from .fuse import merge_op_dag
from .opgraph import build_op_dag

_backward_programs = {}


def _backward_program(dag, opt_level, math):
    key = (dag.text(), opt_level >= 3, math)
    hit = _backward_programs.get(key)
    if hit is None:
        bdag, has_grad = compose_backward(dag)
        if any(has_grad):
            fused = merge_op_dag(bdag) if opt_level >= 3 else bdag
            hit = (runtime.Program(fused, math), has_grad)
        else:
            hit = (None, has_grad)
        _backward_programs[key] = hit
    return hit


# ---------------------------------------------------------------------------------------------------------
# The custom operators.  A compiled operator graph is registered under an integer handle; two operators of the
# `ovl_b200` namespace run a graph forward and run its backward graph.  Both are ordinary dispatcher operators
# (`torch.ops.ovl_b200.run`, `torch.ops.ovl_b200.run_backward`) with fake-tensor implementations, so graphs that
# contain them can be traced and exported; autograd is attached with `register_autograd`.
_registry = []          # handle -> (forward Program, op DAG, opt_level, output TensorTypes)
_handles = {}
_ops = None


def _register(prog, dag, opt_level):
    key = (dag.text(), opt_level >= 3, prog.math)
    if key not in _handles:
        out_types = [prog.plans[o].out_types[k] for o, k in prog.dag.outputs]
        _registry.append((prog, dag, opt_level, out_types))
        _handles[key] = len(_registry) - 1
    return _handles[key]


def _define_ops():
    """Create the two custom operators on first use (torch is imported lazily by this package)."""
    global _ops
    if _ops is not None:
        return _ops
    import torch
    from typing import List

    def _device_of(tensors):
        return tensors[0].device.index if tensors else torch.cuda.current_device()

    @torch.library.custom_op('ovl_b200::run', mutates_args=())
    def run(inputs: List[torch.Tensor], handle: int) -> List[torch.Tensor]:
        prog = _registry[handle][0]
        device = _device_of(inputs)
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream().cuda_stream
            outs, _ = prog.run([x.contiguous() for x in inputs], device, stream, None)
        return list(outs)

    @run.register_fake
    def _(inputs, handle):
        out_types = _registry[handle][3]
        dev = inputs[0].device if inputs else 'cuda'
        return [torch.empty(tuple(t.shape), dtype=t.dtype.as_torch(), device=dev) for t in out_types]

    @torch.library.custom_op('ovl_b200::run_backward', mutates_args=())
    def run_backward(inputs: List[torch.Tensor], grads: List[torch.Tensor], handle: int) -> List[torch.Tensor]:
        prog, dag, opt_level, _ = _registry[handle]
        bprog, has_grad = _backward_program(dag, opt_level, prog.math)
        device = _device_of(inputs)
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream().cuda_stream
            outs, _ = bprog.run([x.contiguous() for x in list(inputs) + list(grads)], device, stream, None)
        return list(outs)

    @run_backward.register_fake
    def _(inputs, grads, handle):
        prog, dag, opt_level, _ = _registry[handle]
        _, has_grad = _backward_program(dag, opt_level, prog.math)
        return [torch.empty_like(x) for x, h in zip(inputs, has_grad) if h]

    def setup_context(ctx, inputs, output):
        tensors, handle = inputs
        ctx.handle = handle
        ctx.save_for_backward(*tensors)

    def backward(ctx, grad_outputs):
        handle = ctx.handle
        prog, dag, opt_level, out_types = _registry[handle]
        bprog, has_grad = _backward_program(dag, opt_level, prog.math)
        saved = list(ctx.saved_tensors)
        if bprog is None:
            return [None for _ in has_grad], None
        grads_in = []
        for g, t, x in zip(grad_outputs, out_types, [None] * len(out_types)):
            if g is None:
                g = torch.zeros(tuple(t.shape), dtype=t.dtype.as_torch(), device=saved[0].device)
            grads_in.append(g)
        outs = iter(torch.ops.ovl_b200.run_backward(saved, grads_in, handle))
        return [next(outs) if h else None for h in has_grad], None

    run.register_autograd(backward, setup_context=setup_context)
    _ops = (run, run_backward)
    return _ops


def as_torch(tensor_list, opt_level=3, math=None):
    """Evaluate operator outputs on the GPU as torch tensors, differentiable with respect to the torch leaf
    inputs that require grad.  A single requested output comes back bare, several as a list
    (as ``as_tensorflow`` does, opveclib/operator.py:2409-2412).  The graph runs as the custom operator
    ``torch.ops.ovl_b200.run``; its backward as ``torch.ops.ovl_b200.run_backward``.  ``math``: the math lowering
    of the forward and backward kernels ('exact', 'tolerance'; None: the current mode)."""
    import torch
    outputs = runtime.as_output_list(tensor_list)
    single = not isinstance(tensor_list, (list, tuple)) and len(outputs) == 1
    prog, dag = runtime.compile_outputs(outputs, opt_level, math)
    if not torch.cuda.is_available():
        raise RuntimeError('opveclib_b200 needs a CUDA device: there is no CPU execution path')
    device = torch.cuda.current_device()
    leaves = []
    for x, t in zip(dag.inputs, dag.input_types):
        if isinstance(x, torch.Tensor):
            if not x.is_cuda:
                raise TypeError('as_torch expects CUDA tensors (or numpy arrays) as operator inputs')
            device = x.device.index
            leaves.append(x)
        else:
            leaves.append(torch.from_numpy(np.ascontiguousarray(x)))
    leaves = [x if x.is_cuda else x.to('cuda:%d' % device) for x in leaves]
    _define_ops()
    handle = _register(prog, dag, opt_level)
    results = list(torch.ops.ovl_b200.run(leaves, handle))
    return results[0] if single or len(results) == 1 else results


def as_tensorflow(tensor_list, opt_level=3):
    """The reference's TensorFlow bridge (opveclib/operator.py:2338-2354) has no counterpart here: this backend
    hands results to PyTorch.  Kept under its old name so that code written for the reference fails with a
    pointer to the replacement instead of an AttributeError."""
    raise NotImplementedError('as_tensorflow is not available in the B200 backend: use as_torch(outputs), which '
                              'returns differentiable torch CUDA tensors')
