"""One-dimensional multi-channel convolution / cross-correlation as an operator that keeps its working set in
worker-local tensors (same interface and results as ``conv_1d`` of opveclib/examples/conv1D.py:18-203).

    out[batch, filter, e] = sum over channels c and taps k of  x[batch, c, first + e + k] * v[filter, c, k']

with k' = k ('as-is', cross-correlation) or taps - 1 - k ('flipped', convolution), samples outside the input
reading as zero, and ``first`` / the number of outputs set by the border mode ('same', 'valid', 'full').  Terms
are accumulated in float64 in channel-major, tap-minor order and the sum is cast to the input type.
"""
from .. import expr as ovl
from ..opgraph import operator

#: consecutive output samples computed by one worker
OUTPUTS_PER_WORKER = 8


@operator()
def conv_1d(x, v, kernel_orientation='as-is', stride=1, mode='same', data_format='NCE'):
    """``x``: [batches, channels, elements], ``v``: [filters, channels, taps], both laid out as ``data_format``
    says (a permutation of 'N', 'C', 'E'; for the filter 'N' is the filter axis).  ``stride`` is validated and
    otherwise has no effect, as in the reference."""
    if kernel_orientation not in ('as-is', 'flipped'):
        raise ValueError("kernel_orientation must be 'as-is' or 'flipped'")
    if x.rank != 3 or v.rank != 3 or sorted(data_format) != ['C', 'E', 'N']:
        raise ValueError('expected rank-3 tensors and a data_format that permutes N, C and E')
    n_ax, c_ax, e_ax = data_format.find('N'), data_format.find('C'), data_format.find('E')
    batches, channels, elements = x.shape[n_ax], x.shape[c_ax], x.shape[e_ax]
    filters, taps = v.shape[n_ax], v.shape[e_ax]
    if v.shape[c_ax] != channels:
        raise ValueError('Channel axis size of input must match that of the filter.')
    if not isinstance(stride, int) or stride < 1 or stride > elements:
        raise ValueError('Stride must be a positive integer')
    left = taps // 2
    if mode in ('same', 'valid') and taps > elements:
        raise ValueError('filter size, %d,  cannot be larger than number of elements, %d' % (taps, elements))
    if mode == 'same':
        first, outputs = -left, elements
    elif mode == 'valid':
        first, outputs = 0, elements - taps + 1
    elif mode == 'full':
        first, outputs = -(taps - 1), elements + taps - 1
    else:
        raise ValueError("mode must be 'same', 'valid', or 'full'.")

    def arranged(n, c, e):
        index = [None, None, None]
        index[n_ax], index[c_ax], index[e_ax] = n, c, e
        return index

    out = ovl.output(arranged(batches, filters, outputs), x.dtype)
    per_worker = OUTPUTS_PER_WORKER
    blocks = (outputs + per_worker - 1) // per_worker
    pos = ovl.position_in([batches, filters, blocks])
    batch, filt = pos[0], pos[1]
    base = ovl.cast(pos[2], ovl.int64) * per_worker          # first output sample of this worker

    window_len = per_worker + taps - 1
    sums = ovl.zeros([per_worker], ovl.float64)
    window = ovl.zeros([window_len], x.dtype)
    weights = ovl.zeros([taps], v.dtype)
    for c in ovl.arange(channels):
        for k in ovl.arange(taps):
            tap = k if kernel_orientation == 'as-is' else (taps - 1) - k
            weights[k] = v[arranged(filt, c, tap)]
        for j in ovl.arange(window_len):
            sample = base + j + first
            with ovl.if_(ovl.logical_and(sample >= 0, sample < elements)):
                window[j] = x[arranged(batch, c, sample)]
            with ovl.else_():
                window[j] = 0
        for e in ovl.arange(per_worker):
            for k in ovl.arange(taps):
                sums[e] = sums[e] + ovl.cast(window[e + k], ovl.float64) * ovl.cast(weights[k], ovl.float64)
    for e in ovl.arange(per_worker):
        with ovl.if_(base + e < outputs):
            out[arranged(batch, filt, base + e)] = ovl.cast(sums[e], out.dtype)
    return out
