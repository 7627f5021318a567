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


def _backward_program(dag, opt_level):
    key = (dag.text(), opt_level >= 3)
    hit = _backward_programs.get(key)
    if hit is None:
        bdag, has_grad = compose_backward(dag)
        if any(has_grad):
            fused = merge_op_dag(bdag) if opt_level >= 3 else bdag
            hit = (runtime.Program(fused), has_grad)
        else:
            hit = (None, has_grad)
        _backward_programs[key] = hit
    return hit


def as_torch(tensor_list, opt_level=3):
    """Evaluate operator outputs on the GPU as torch tensors, differentiable with respect to the torch leaf
    inputs that require grad.  A single requested output comes back bare, several as a list
    (as ``as_tensorflow`` does, opveclib/operator.py:2409-2412)."""
    import torch
    single = not isinstance(tensor_list, (list, tuple))
    outputs = [tensor_list] if single else list(tensor_list)
    prog, dag = runtime.compile_outputs(outputs, opt_level)
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
    out_types = [prog.plans[o].out_types[k] for o, k in prog.dag.outputs]

    class _OvlFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *inputs):
            with torch.cuda.device(device):
                stream = torch.cuda.current_stream().cuda_stream
                staged = [x.detach().contiguous() for x in inputs]
                outs, _ = prog.run(staged, device, stream, None)
            ctx.save_for_backward(*staged)
            ctx.mark_non_differentiable(*[o for o, t in zip(outs, out_types) if not t.dtype.is_float])
            return tuple(outs)

        @staticmethod
        def backward(ctx, *grad_outputs):
            bprog, has_grad = _backward_program(dag, opt_level)
            if bprog is None:
                return tuple(None for _ in has_grad)
            saved = list(ctx.saved_tensors)
            grads_in = []
            for g, t in zip(grad_outputs, out_types):
                if g is None:
                    g = torch.zeros(t.shape, dtype=t.dtype.as_torch(), device='cuda:%d' % device)
                grads_in.append(g.contiguous())
            with torch.cuda.device(device):
                stream = torch.cuda.current_stream().cuda_stream
                outs, _ = bprog.run(saved + grads_in, device, stream, None)
            it = iter(outs)
            return tuple(next(it) if h else None for h in has_grad)

    results = _OvlFunction.apply(*leaves)
    results = list(results)
    return results[0] if single or len(results) == 1 else results


def as_tensorflow(tensor_list, opt_level=3):
    """The reference's TensorFlow bridge (opveclib/operator.py:2338-2354) has no counterpart here: this backend
    hands results to PyTorch.  Kept under its old name so that code written for the reference fails with a
    pointer to the replacement instead of an AttributeError."""
    raise NotImplementedError('as_tensorflow is not available in the B200 backend: use as_torch(outputs), which '
                              'returns differentiable torch CUDA tensors')
