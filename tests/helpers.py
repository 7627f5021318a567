"""Comparison helpers shared by the test modules."""
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
DRYRUN = bool(os.environ.get('OVL_B200_DRYRUN'))


def load_golden(name):
    data = np.load(os.path.join(GOLDEN_DIR, name + '.npz'))
    ins = [data['in_%d' % i] for i in range(sum(1 for k in data.files if k.startswith('in_')))]
    outs = [data['out_%d' % i] for i in range(sum(1 for k in data.files if k.startswith('out_')))]
    return ins, outs


def ulp_diff(a, b):
    """Distance in units in the last place between two float arrays of the same dtype (NaNs must coincide)."""
    a = np.asarray(a)
    b = np.asarray(b)
    assert a.dtype == b.dtype and a.shape == b.shape
    nan = np.isnan(a) | np.isnan(b)
    assert np.array_equal(np.isnan(a), np.isnan(b)), 'NaN pattern differs'
    it = np.int32 if a.dtype == np.float32 else np.int64
    ia = a.view(it).astype(np.int64)
    ib = b.view(it).astype(np.int64)
    # map the sign-magnitude float ordering onto a monotonic integer line
    top = np.int64(1) << (31 if a.dtype == np.float32 else 63)
    ia = np.where(ia < 0, -(ia + top) if a.dtype == np.float32 else -(ia ^ np.int64(-2 ** 63)), ia)
    ib = np.where(ib < 0, -(ib + top) if a.dtype == np.float32 else -(ib ^ np.int64(-2 ** 63)), ib)
    d = np.abs(ia - ib)
    d[nan] = 0
    return d


def assert_exact(got, want, what=''):
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.dtype == want.dtype, '%s dtype %s != %s' % (what, got.dtype, want.dtype)
    assert got.shape == want.shape, '%s shape %s != %s' % (what, got.shape, want.shape)
    if not np.array_equal(got, want, equal_nan=got.dtype.kind == 'f'):
        bad = np.flatnonzero(~((got == want) | ((got != got) & (want != want))).reshape(-1))
        raise AssertionError('%s: %d of %d elements differ, first at %d: got %r want %r' % (
            what, bad.size, got.size, bad[0], got.reshape(-1)[bad[0]], want.reshape(-1)[bad[0]]))


def assert_close(got, want, rtol, atol=0.0, what=''):
    """|got - want| <= atol + rtol * |want| element-wise; infinities and NaNs must coincide."""
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.dtype == want.dtype, '%s dtype %s != %s' % (what, got.dtype, want.dtype)
    assert got.shape == want.shape, '%s shape %s != %s' % (what, got.shape, want.shape)
    if got.dtype.kind != 'f':
        return assert_exact(got, want, what)
    g = got.astype(np.float64)
    w = want.astype(np.float64)
    finite = np.isfinite(w)
    assert np.array_equal(finite, np.isfinite(g)), what + ': finite pattern differs'
    assert np.array_equal(g[~finite], w[~finite], equal_nan=True), what + ': inf/nan values differ'
    err = np.abs(g - w)[finite]
    lim = (atol + rtol * np.abs(w))[finite] if np.ndim(atol) else atol + rtol * np.abs(w[finite])
    if np.any(err > lim):
        i = int(np.argmax(err - lim))
        raise AssertionError('%s: %d of %d elements outside rtol=%g atol=%s; worst |diff|=%g at value %g' % (
            what, int(np.sum(err > lim)), err.size, rtol, np.max(atol), err[i], w[finite][i]))
