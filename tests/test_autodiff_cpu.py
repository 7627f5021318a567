"""Backward operator graphs composed from ``@gradient`` definitions, checked on the CPU through the oracle.

The reference checks its merged gradient graphs against TensorFlow's autodiff
(opveclib/test/test_operator_merge.py:395-483, opveclib/stdops/test_math.py:91-157, 270-307); torch's autograd
in float64 plays that role here."""
import numpy as np
import torch

import cases
from helpers import assert_exact
from opveclib_b200.autodiff import compose_backward
from opveclib_b200.fuse import merge_op_dag
from opveclib_b200.opgraph import build_op_dag
from oracle import runner


def _run_backward(dag, grads_out):
    bdag, has_grad = compose_backward(dag)
    fused = merge_op_dag(bdag)
    leaves = list(dag.inputs) + list(grads_out)
    bdag.inputs = leaves
    fused.inputs = leaves
    plain, _ = runner.run_dag(bdag)
    merged, _ = runner.run_dag(fused)
    for a, b in zip(plain, merged):
        assert_exact(b, a, 'fused backward')
    return plain, has_grad, len(bdag.kernels), len(fused.kernels)


def test_stdops_lstm_backward_matches_autograd_and_fuses_to_one_kernel():
    ns = cases.impl()
    so = ns.stdops
    rs = np.random.RandomState(0)
    g, c = rs.normal(size=(4, 24)), rs.normal(size=(4, 6))
    i, j, f, o = so.split(g, split_dim=1, num_split=4)
    new_c = so.mul(c, so.sigmoid(f)) + so.sigmoid(i) * so.tanh(j)
    new_h = so.tanh(new_c) * so.sigmoid(o)
    dag = build_op_dag(new_c, new_h)
    dc, dh = rs.normal(size=(4, 6)), rs.normal(size=(4, 6))
    grads, has_grad, n_plain, n_fused = _run_backward(dag, [dc, dh])
    assert has_grad == [True, True] and n_plain > 10 and n_fused == 1

    tg = torch.tensor(g, requires_grad=True)
    tc = torch.tensor(c, requires_grad=True)
    ti, tj, tf, to = tg.chunk(4, dim=1)
    nc = tc * torch.sigmoid(tf) + torch.sigmoid(ti) * torch.tanh(tj)
    nh = torch.tanh(nc) * torch.sigmoid(to)
    ((nc * torch.tensor(dc)).sum() + (nh * torch.tensor(dh)).sum()).backward()
    want = {id(g): tg.grad.numpy(), id(c): tc.grad.numpy()}
    for leaf, got in zip(dag.inputs, grads):
        np.testing.assert_allclose(got, want[id(leaf)], rtol=1e-12, atol=1e-14)


def test_hand_fused_lstm_gradient_operator_is_used():
    ns = cases.impl()
    rs = np.random.RandomState(1)
    g, c = rs.normal(size=(3, 16)), rs.normal(size=(3, 4))
    op = ns.lstm(g, c, forget_bias=0.5)
    dag = build_op_dag(op[0], op[1])
    dc, dh = rs.normal(size=(3, 4)), rs.normal(size=(3, 4))
    grads, has_grad, n_plain, n_fused = _run_backward(dag, [dc, dh])
    assert has_grad == [True, True] and n_plain == 1     # only lstm_grad is needed: it recomputes what it uses

    tg = torch.tensor(g, requires_grad=True)
    tc = torch.tensor(c, requires_grad=True)
    ti, tj, tf, to = tg.chunk(4, dim=1)
    nc = tc * torch.sigmoid(tf + 0.5) + torch.sigmoid(ti) * torch.tanh(tj)
    nh = torch.tanh(nc) * torch.sigmoid(to)
    ((nc * torch.tensor(dc)).sum() + (nh * torch.tensor(dh)).sum()).backward()
    want = {id(g): tg.grad.numpy(), id(c): tc.grad.numpy()}
    for leaf, got in zip(dag.inputs, grads):
        np.testing.assert_allclose(got, want[id(leaf)], rtol=1e-10, atol=1e-12)


def test_shared_input_contributions_are_summed_and_missing_gradients_block():
    ns = cases.impl()
    so = ns.stdops
    rs = np.random.RandomState(2)
    x, y = rs.uniform(0.5, 2, 7), rs.uniform(0.5, 2, 7)
    z = so.mul(x, y) + so.div(x, y) - ns.expm1(x)      # x feeds three operators
    dag = build_op_dag(z)
    dz = rs.normal(size=7)
    grads, has_grad, _, _ = _run_backward(dag, [dz])
    want = {id(x): dz * (y + 1 / y - np.exp(x)), id(y): dz * (x - x / (y * y))}
    for leaf, got in zip(dag.inputs, grads):
        np.testing.assert_allclose(got, want[id(leaf)], rtol=1e-12)
    # `mod` has no gradient: nothing flows to its inputs
    w = so.mod(x, y) * y
    dag = build_op_dag(w)
    bdag, has_grad = compose_backward(dag)
    flags = dict((id(leaf), h) for leaf, h in zip(dag.inputs, has_grad))
    assert flags[id(x)] is False


def test_custom_operators_are_registered_with_fake_tensor_support():
    """`as_torch` runs graphs as `torch.ops.ovl_b200.run` / `run_backward`; both can be traced without a device
    (shapes and dtypes come from the compiled graph's signature)."""
    import numpy as np
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode
    import cases
    from opveclib_b200 import runtime, torch_bridge
    ns = cases.impl()
    g, c = np.zeros((6, 32), np.float32), np.zeros((6, 8), np.float32)
    op = ns.lstm(g, c, forget_bias=0.0)
    prog, dag = runtime.compile_outputs([op[0], op[1]])
    torch_bridge._define_ops()
    handle = torch_bridge._register(prog, dag, 3)
    assert handle == torch_bridge._register(prog, dag, 3)
    assert str(torch.ops.ovl_b200.run.default._schema).startswith('ovl_b200::run(Tensor[] inputs')
    with FakeTensorMode():
        a, b = torch.empty((6, 32), device='cuda'), torch.empty((6, 8), device='cuda')
        outs = torch.ops.ovl_b200.run([a, b], handle)
        assert [tuple(o.shape) for o in outs] == [(6, 8), (6, 8)] and outs[0].dtype == torch.float32
        grads = torch.ops.ovl_b200.run_backward([a, b], list(outs), handle)
        assert [tuple(x.shape) for x in grads] == [(6, 32), (6, 8)]


def _torch_grads(fn, arrays, grads_out):
    leaves = [torch.tensor(a, requires_grad=True) for a in arrays]
    outs = fn(*leaves)
    outs = outs if isinstance(outs, (list, tuple)) else [outs]
    total = sum((o * torch.tensor(g)).sum() for o, g in zip(outs, grads_out))
    total.backward()
    return [x.grad.numpy() if x.grad is not None else None for x in leaves]


def test_stdops_binary_and_unary_gradients_match_autograd():
    """The component-wise gradients of the operator library (the reference compares them with TensorFlow's,
    opveclib/stdops/test_math.py:91-157)."""
    so = cases.impl().stdops
    rs = np.random.RandomState(11)
    lhs = rs.random_sample(100)
    rhs = lhs + rs.randint(-1, 2, size=100) + 0.25          # (never zero: it is also used as a divisor)
    above = rs.random_sample(100)
    for fcn, ref in [(so.add, torch.add), (so.sub, torch.sub), (so.mul, torch.mul), (so.div, torch.div)]:
        for a, b in ((lhs, rhs), (rhs, lhs)):
            dag = build_op_dag(fcn(a, b))
            grads, has_grad, _, _ = _run_backward(dag, [above])
            want = dict(zip((id(a), id(b)), _torch_grads(ref, [a, b], [above])))
            assert has_grad == [True, True]
            for leaf, got in zip(dag.inputs, grads):
                np.testing.assert_allclose(got, want[id(leaf)], rtol=1e-13, atol=0)
    arg = rs.random_sample(100)
    for fcn, ref in [(so.neg, torch.neg), (so.tanh, torch.tanh), (so.sin, torch.sin), (so.cos, torch.cos),
                     (so.tan, torch.tan), (so.sigmoid, torch.sigmoid)]:
        dag = build_op_dag(fcn(arg))
        grads, has_grad, _, _ = _run_backward(dag, [above])
        np.testing.assert_allclose(grads[0], _torch_grads(ref, [arg], [above])[0], rtol=1e-12, atol=1e-15)


def test_split_and_concat_gradients_match_autograd():
    """Gradients through split and concat of equal parts (opveclib/stdops/test_math.py:159-268)."""
    so = cases.impl().stdops
    rs = np.random.RandomState(12)
    x = rs.random_sample((3, 8, 5))
    parts = so.split(x, split_dim=1, num_split=4)
    outs = [so.mul(parts[0], parts[3]), so.add(parts[1], parts[2])]
    dag = build_op_dag(*outs)
    above = [rs.random_sample((3, 2, 5)), rs.random_sample((3, 2, 5))]
    grads, has_grad, _, _ = _run_backward(dag, above)

    def ref(t):
        p = t.chunk(4, dim=1)
        return [p[0] * p[3], p[1] + p[2]]
    np.testing.assert_allclose(grads[0], _torch_grads(ref, [x], above)[0], rtol=1e-13, atol=0)

    a, b, c = rs.random_sample((4, 3)), rs.random_sample((4, 3)), rs.random_sample((4, 3))
    cat = so.concat(a, b, c, concat_dim=1)
    dag = build_op_dag(so.mul(cat, cat))
    above = [rs.random_sample((4, 9))]
    grads, has_grad, _, _ = _run_backward(dag, above)
    want = dict(zip((id(a), id(b), id(c)),
                    _torch_grads(lambda p, q, r: torch.cat([p, q, r], dim=1) ** 2, [a, b, c], above)))
    assert has_grad == [True, True, True]
    for leaf, got in zip(dag.inputs, grads):
        np.testing.assert_allclose(got, want[id(leaf)], rtol=1e-13, atol=0)
