"""Generic accumulation along one axis, and the cumsum / cumprod built on it.

Same algorithm as opveclib/examples/test_accumulate.py:22-147: one worker per position of the tensor with the
accumulation axis removed (a rank-1 tensor has a single worker); the worker seeds an accumulator with the first
element along the axis, stores it, then walks the rest of the axis applying ``inner_fcn(accum, x)`` and storing
each running value.  The B200 backend recognises this loop as a scan and runs it as a cooperative parallel
scan instead of one serial thread per line.
"""
from .. import expr as ovl
from ..opgraph import operator


@operator()
def accumulate(x, inner_fcn=None, axis=None):
    """Accumulate ``inner_fcn`` along ``axis`` of ``x`` (inclusive).  ``inner_fcn`` and ``axis`` are constants
    and must be passed by keyword."""
    assert isinstance(axis, int)
    assert 0 <= axis < x.rank

    if x.rank == 1:
        workgroup_shape = [1]
    else:
        workgroup_shape = [n for d, n in enumerate(x.shape) if d != axis]
    pos = ovl.position_in(workgroup_shape)
    out = ovl.output_like(x)

    def at(axis_index):
        # tensor index of the element `axis_index` along the axis, on this worker's line
        index, skipped = [], 0
        for d in range(x.rank):
            if d == axis:
                index.append(axis_index)
                skipped = 1
            else:
                index.append(pos[d - skipped])
        return index

    accum = ovl.variable(x[at(0)], x.dtype)
    out[at(0)] = accum
    for i in ovl.arange(1, x.shape[axis]):
        accum <<= inner_fcn(accum, x[at(i)])
        out[at(i)] = accum
    return out


def cumsum(x, axis=0):
    """Cumulative sum along ``axis`` (numpy.cumsum semantics)."""
    return accumulate(x, inner_fcn=lambda a, b: a + b, axis=axis)


def cumprod(x, axis=0):
    """Cumulative product along ``axis`` (numpy.cumprod semantics)."""
    return accumulate(x, inner_fcn=lambda a, b: a * b, axis=axis)
