"""log(1 + x) that stays accurate for tiny |x| (algorithm of opveclib/examples/test_log1p.py:22-79)."""
from .. import expr as ovl
from ..opgraph import operator, gradient


@operator()
def log1p(x):
    """Element-wise log(1 + x).  With u = 1 + x and d = u - 1: +inf passes through; d == 0 gives x;
    otherwise log(u) * x / d compensates the rounding of u."""
    out = ovl.output_like(x)
    pos = ovl.position_in(x.shape)
    u = 1.0 + x[pos]
    d = u - 1.0
    with ovl.if_(ovl.logical_and(ovl.isinf(x[pos]), x[pos] > 0.0)):
        out[pos] = x[pos]
    with ovl.elif_(d == 0):
        out[pos] = x[pos]
    with ovl.else_():
        out[pos] = ovl.log(u) * x[pos] / d
    return out


@gradient(log1p)
@operator()
def log1p_grad(x, grad):
    """d/dx log1p = 1 / (x + 1), times the incoming gradient."""
    out = ovl.output(x.shape, x.dtype)
    pos = ovl.position_in(x.shape)
    out[pos] = 1.0 / (x[pos] + 1.0) * grad[pos]
    return out
