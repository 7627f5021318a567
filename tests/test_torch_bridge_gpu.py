"""The torch bridge on a GPU: torch tensors in and out, gradients through ``torch.autograd``."""
import numpy as np
import pytest

import cases
from helpers import DRYRUN

pytestmark = pytest.mark.gpu


def _cuda(a, grad=False):
    import torch
    if DRYRUN:
        return a
    return torch.tensor(a, device='cuda', requires_grad=grad)


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_as_torch_forward_and_backward_match_autograd():
    import torch
    ns = cases.impl()
    so = ns.stdops
    rs = np.random.RandomState(3)
    g = torch.tensor(rs.normal(size=(8, 64)).astype(np.float32), device='cuda', requires_grad=True)
    c = torch.tensor(rs.normal(size=(8, 16)).astype(np.float32), device='cuda', requires_grad=True)
    i, j, f, o = so.split(g, split_dim=1, num_split=4)
    new_c = so.mul(c, so.sigmoid(f)) + so.sigmoid(i) * so.tanh(j)
    new_h = so.tanh(new_c) * so.sigmoid(o)
    nc, nh = ns.ovl.as_torch([new_c, new_h])
    assert nc.is_cuda and nc.requires_grad
    wc = torch.tensor(rs.normal(size=(8, 16)).astype(np.float32), device='cuda')
    wh = torch.tensor(rs.normal(size=(8, 16)).astype(np.float32), device='cuda')
    ((nc * wc).sum() + (nh * wh).sum()).backward()
    got_g, got_c = g.grad.clone(), c.grad.clone()

    g2 = g.detach().clone().requires_grad_(True)
    c2 = c.detach().clone().requires_grad_(True)
    ti, tj, tf, to = g2.chunk(4, dim=1)
    rc = c2 * torch.sigmoid(tf) + torch.sigmoid(ti) * torch.tanh(tj)
    rh = torch.tanh(rc) * torch.sigmoid(to)
    ((rc * wc).sum() + (rh * wh).sum()).backward()
    torch.testing.assert_close(nc.detach(), rc.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(nh.detach(), rh.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(got_g, g2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(got_c, c2.grad, rtol=1e-4, atol=1e-5)


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_hand_fused_lstm_through_as_torch_and_evaluate_on_device_tensors():
    import torch
    ns = cases.impl()
    rs = np.random.RandomState(4)
    g = torch.tensor(rs.normal(size=(16, 128)).astype(np.float32), device='cuda', requires_grad=True)
    c = torch.tensor(rs.normal(size=(16, 32)).astype(np.float32), device='cuda', requires_grad=True)
    op = ns.lstm(g, c, forget_bias=0.0)
    nc, nh = ns.ovl.as_torch([op[0], op[1]])
    (nc.sum() + 2 * nh.sum()).backward()
    g2 = g.detach().clone().requires_grad_(True)
    c2 = c.detach().clone().requires_grad_(True)
    ti, tj, tf, to = g2.chunk(4, dim=1)
    rc = c2 * torch.sigmoid(tf) + torch.sigmoid(ti) * torch.tanh(tj)
    rh = torch.tanh(rc) * torch.sigmoid(to)
    (rc.sum() + 2 * rh.sum()).backward()
    torch.testing.assert_close(g.grad, g2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(c.grad, c2.grad, rtol=1e-4, atol=1e-5)
    # evaluate() with device tensors keeps results on the device
    out = ns.ovl.evaluate([op[0], op[1]])
    assert all(isinstance(t, torch.Tensor) and t.is_cuda for t in out)
    torch.testing.assert_close(out[0], rc.detach(), rtol=1e-5, atol=1e-6)


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_as_torch_with_the_tolerance_lowering():
    """``as_torch(..., math='tolerance')``: forward and backward graphs are both generated with the tolerance
    lowering (a handle of its own: the exact graph of the same operators is untouched) and agree with torch."""
    import torch
    from opveclib_b200 import torch_bridge
    ns = cases.impl()
    rs = np.random.RandomState(6)
    g = torch.tensor(rs.normal(size=(16, 128)).astype(np.float32), device='cuda', requires_grad=True)
    c = torch.tensor(rs.normal(size=(16, 32)).astype(np.float32), device='cuda', requires_grad=True)
    op = ns.lstm(g, c, forget_bias=0.0)
    handles_before = len(torch_bridge._registry)
    nc_exact, _ = ns.ovl.as_torch([op[0], op[1]], math='exact')
    nc, nh = ns.ovl.as_torch([op[0], op[1]], math='tolerance')
    # (the exact graph of these operators may have a handle from an earlier call; the tolerance one is new)
    assert handles_before + 1 <= len(torch_bridge._registry) <= handles_before + 2
    assert torch_bridge._registry[-1][0].math == 'tolerance'
    assert torch_bridge._registry[-1][0].plans[0].meta['vec']['paired']
    (nc.sum() + 2 * nh.sum()).backward()
    g2 = g.detach().clone().requires_grad_(True)
    c2 = c.detach().clone().requires_grad_(True)
    ti, tj, tf, to = g2.chunk(4, dim=1)
    rc = c2 * torch.sigmoid(tf) + torch.sigmoid(ti) * torch.tanh(tj)
    rh = torch.tanh(rc) * torch.sigmoid(to)
    (rc.sum() + 2 * rh.sum()).backward()
    torch.testing.assert_close(nc.detach(), rc.detach(), rtol=1e-5, atol=2e-6)
    torch.testing.assert_close(nc.detach(), nc_exact.detach(), rtol=1e-5, atol=2e-6)
    torch.testing.assert_close(g.grad, g2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(c.grad, c2.grad, rtol=1e-4, atol=1e-5)


def test_backward_kernels_compile():
    """Cache warming for the two tests above (also runs without a device): trace, compose, fuse, compile."""
    from opveclib_b200 import runtime
    from opveclib_b200.autodiff import compose_backward
    from opveclib_b200.fuse import merge_op_dag
    from opveclib_b200.opgraph import build_op_dag
    ns = cases.impl()
    so = ns.stdops
    g, c = np.zeros((8, 64), np.float32), np.zeros((8, 16), np.float32)
    i, j, f, o = so.split(g, split_dim=1, num_split=4)
    new_c = so.mul(c, so.sigmoid(f)) + so.sigmoid(i) * so.tanh(j)
    new_h = so.tanh(new_c) * so.sigmoid(o)
    g2, c2 = np.zeros((16, 128), np.float32), np.zeros((16, 32), np.float32)
    op = ns.lstm(g2, c2, forget_bias=0.0)
    for outs in ([new_c, new_h], [op[0], op[1]]):
        runtime.compile_outputs(outs)
        bdag, _ = compose_backward(build_op_dag(*outs))
        prog = runtime.Program(merge_op_dag(bdag))
        assert len(prog.plans) == 1


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_the_reference_gradient_examples_against_torch_autograd():
    """The two cases of opveclib/test/test_gradients.py (there against TensorFlow's gradients, exact equality):
    z = x*x + 3*y with its hand-written gradient, and a clip operator whose gradient masks the clipped elements."""
    import torch
    ovl = cases.impl().ovl

    @ovl.operator()
    def func(x, y):
        pos = ovl.position_in(x.shape)
        z = ovl.output_like(x)
        z[pos] = x[pos] * x[pos] + 3 * y[pos]
        return z

    @ovl.gradient(func)
    @ovl.operator()
    def func_grad(x, y, dz):
        pos = ovl.position_in(x.shape)
        dx, dy = ovl.output_like(x), ovl.output_like(y)
        dx[pos] = 2.0 * x[pos] * dz[pos]
        dy[pos] = 3.0 * dz[pos]
        return dx, dy

    @ovl.operator()
    def clip(arg, threshold1=None, threshold2=None):
        pos = ovl.position_in(arg.shape)
        clipped = ovl.output_like(arg)
        x = arg[pos]
        with ovl.if_(x < threshold1):
            clipped[pos] = threshold1
        with ovl.elif_(x > threshold2):
            clipped[pos] = threshold2
        with ovl.else_():
            clipped[pos] = x
        return clipped

    @ovl.gradient(clip)
    @ovl.operator()
    def clip_grad(arg, d_arg, threshold1=None, threshold2=None):
        pos = ovl.position_in(arg.shape)
        g = ovl.output_like(arg)
        x = arg[pos]
        with ovl.if_(x < threshold1):
            g[pos] = 0
        with ovl.elif_(x > threshold2):
            g[pos] = 0
        with ovl.else_():
            g[pos] = d_arg[pos]
        return g

    rs = np.random.RandomState(5)
    a = torch.tensor(rs.random_sample(10), device='cuda', requires_grad=True)
    b = torch.tensor(rs.random_sample(10), device='cuda', requires_grad=True)
    above = torch.tensor(rs.random_sample(10), device='cuda')
    z = ovl.as_torch(func(a, b))
    z.backward(above)
    a2, b2 = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    (a2 * a2 + 3 * b2).backward(above)
    assert torch.equal(z.detach(), (a2 * a2 + 3 * b2).detach())
    assert torch.equal(a.grad, a2.grad) and torch.equal(b.grad, b2.grad)

    c = torch.tensor(rs.random_sample(10), device='cuda', requires_grad=True)
    scale = float(rs.random_sample(1)[0])
    (ovl.as_torch(clip(c, threshold1=0.1, threshold2=0.9)).sum() * scale).backward()
    c2 = c.detach().clone().requires_grad_(True)
    (torch.clamp(c2, 0.1, 0.9).sum() * scale).backward()
    assert torch.equal(c.grad, c2.grad)
