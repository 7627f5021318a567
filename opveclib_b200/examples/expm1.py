"""exp(x) - 1 that stays accurate for tiny |x| (algorithm of opveclib/examples/test_expm1.py:22-80)."""
from .. import expr as ovl
from ..opgraph import operator, gradient


@operator()
def expm1(x):
    """Element-wise exp(x) - 1.  +inf passes through; where exp(x) rounds to 1 the result is x; where
    exp(x) - 1 rounds to -1 the result is -1; otherwise (e - 1) * x / log(e) cancels the rounding of e."""
    out = ovl.output_like(x)
    pos = ovl.position_in(x.shape)
    e = ovl.exp(x[pos])
    with ovl.if_(ovl.logical_and(ovl.isinf(x[pos]), x[pos] > 0.0)):
        out[pos] = x[pos]
    with ovl.elif_(e == 1.0):
        out[pos] = x[pos]
    with ovl.elif_((e - 1.0) == -1.0):
        out[pos] = -1.0
    with ovl.else_():
        out[pos] = (e - 1.0) * x[pos] / ovl.log(e)
    return out


@gradient(expm1)
@operator()
def expm1_grad(x, grad):
    """d/dx expm1 = exp(x), times the incoming gradient."""
    out = ovl.output(x.shape, x.dtype)
    pos = ovl.position_in(x.shape)
    out[pos] = ovl.exp(x[pos]) * grad[pos]
    return out
