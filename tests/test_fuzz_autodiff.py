"""Random graphs of operator-library functions, differentiated: the backward graph composed from the operators'
own gradient definitions must not change a bit under fusion and must agree with torch's autograd in float64
(the reference checks its composed gradients against TensorFlow's, opveclib/stdops/test_math.py:91-307 and
opveclib/test/test_operator_merge.py:395-483)."""
import numpy as np
import pytest
import torch

import cases
from helpers import DRYRUN, assert_exact
from opveclib_b200.autodiff import compose_backward
from opveclib_b200.fuse import merge_op_dag
from opveclib_b200.opgraph import build_op_dag
from oracle import runner

UNARY = ['neg', 'tanh', 'sigmoid', 'sin', 'cos']
BINARY = ['add', 'sub', 'mul', 'div']


def _random_graph(so, seed, wrap=None):
    """The same random function twice: on operator-library values and on torch tensors.  ``wrap`` turns the numpy
    leaves into what the operator library sees (device tensors in the GPU test)."""
    rs = np.random.RandomState(seed)
    rows, cols = int(rs.choice([1, 3, 4, 7])), int(rs.choice([2, 4, 6, 12]))
    leaves = [rs.uniform(0.5, 1.5, (rows, cols)) for _ in range(rs.randint(1, 4))]
    tleaves = [torch.tensor(x, requires_grad=True) for x in leaves]
    if wrap is not None:
        leaves = [wrap(x) for x in leaves]
    values = [(x, t) for x, t in zip(leaves, tleaves)]          # all of shape [rows, cols]
    for _ in range(rs.randint(3, 10)):
        kind = rs.choice(['unary', 'binary', 'binary', 'splitcat'])
        pick = lambda: values[rs.randint(len(values))]     # noqa: E731
        if kind == 'unary':
            name = str(rs.choice(UNARY))
            a, ta = pick()
            values.append((getattr(so, name)(a), getattr(torch, name)(ta)))
        elif kind == 'binary':
            name = str(rs.choice(BINARY))
            (a, ta), (b, tb) = pick(), pick()
            if name == 'div':
                # keep the divisor away from zero: 2 + tanh(.) lies in (1, 3)
                b, tb = so.add(so.tanh(b), np.full((rows, cols), 2.0)), torch.tanh(tb) + 2.0
            values.append((getattr(so, name)(a, b), getattr(torch, name)(ta, tb)))
        else:
            # split along the columns, combine the halves, put them together again
            (a, ta), (b, tb) = pick(), pick()
            a0, a1 = so.split(a, split_dim=1, num_split=2)
            ta0, ta1 = ta.chunk(2, dim=1)
            b0, b1 = so.split(b, split_dim=1, num_split=2)
            tb0, tb1 = tb.chunk(2, dim=1)
            values.append((so.concat(so.mul(a0, b1), so.sub(a1, b0), concat_dim=1),
                           torch.cat([ta0 * tb1, ta1 - tb0], dim=1)))
    produced = values[len(leaves):]
    outs = [produced[-1]] + ([produced[rs.randint(len(produced) - 1)]] if len(produced) > 1 and rs.rand() < 0.5 else [])
    above = [rs.normal(size=(rows, cols)) for _ in outs]
    return leaves, tleaves, [o for o, _ in outs], [t for _, t in outs], above


@pytest.mark.parametrize('seed', range(30))
def test_composed_gradients_match_autograd_and_survive_fusion(seed):
    so = cases.impl().stdops
    leaves, tleaves, outs, touts, above = _random_graph(so, seed)
    dag = build_op_dag(*outs)
    bdag, has_grad = compose_backward(dag)
    fused = merge_op_dag(bdag)
    feed = list(dag.inputs) + list(above)
    bdag.inputs = feed
    fused.inputs = feed
    plain, _ = runner.run_dag(bdag)
    merged, _ = runner.run_dag(fused)
    assert len(fused.kernels) <= len(bdag.kernels)
    for a, b in zip(plain, merged):
        assert_exact(b, a, 'seed %d: fused backward' % seed)

    sum((t * torch.tensor(g)).sum() for t, g in zip(touts, above)).backward()
    want = dict((id(x), t.grad) for x, t in zip(leaves, tleaves))
    grads = iter(plain)
    for leaf, flag in zip(dag.inputs, has_grad):
        if id(leaf) not in want:
            if flag:
                next(grads)             # a constant fed in by the test (the divisor's offset)
            continue
        assert flag
        got = next(grads)
        expect = want[id(leaf)]
        expect = np.zeros_like(leaf) if expect is None else expect.numpy()
        np.testing.assert_allclose(got, expect, rtol=1e-9, atol=1e-11, err_msg='seed %d' % seed)


GPU_SEEDS = range(12)


@pytest.mark.gpu
@pytest.mark.parametrize('seed', GPU_SEEDS)
def test_gradients_through_as_torch_match_autograd(seed):
    """The same graphs on the device: forward through `as_torch`, backward through `torch.autograd` into the fused
    backward kernel, against torch's own autograd of the same function on the CPU."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    so = ns.stdops
    if DRYRUN:
        # cache warming without a device: trace, compose, fuse, compile
        _, _, outs, _, _ = _random_graph(so, seed)
        runtime.compile_outputs(outs)
        bdag, has_grad = compose_backward(build_op_dag(*outs))
        if any(has_grad):
            runtime.Program(merge_op_dag(bdag))
        return
    wrap = lambda x: torch.tensor(x, device='cuda', requires_grad=True)     # noqa: E731
    leaves, tleaves, outs, touts, above = _random_graph(so, seed, wrap)
    results = ns.ovl.as_torch(outs)
    results = results if isinstance(results, (list, tuple)) else [results]
    for got, want in zip(results, touts):
        np.testing.assert_allclose(got.detach().cpu().numpy(), want.detach().numpy(), rtol=1e-11, atol=1e-12)
    sum((r * torch.tensor(g, device='cuda')).sum() for r, g in zip(results, above)).backward()
    sum((t * torch.tensor(g)).sum() for t, g in zip(touts, above)).backward()
    for leaf, ref in zip(leaves, tleaves):
        if ref.grad is None:
            assert leaf.grad is None or not leaf.grad.abs().sum().item()
            continue
        np.testing.assert_allclose(leaf.grad.cpu().numpy(), ref.grad.numpy(), rtol=1e-9, atol=1e-11,
                                   err_msg='seed %d' % seed)
