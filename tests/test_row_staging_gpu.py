"""Per-worker loops over the worker's own row of an input (row sums, row maxima, short dot products): the rows of a
block's workers are staged in shared memory with coalesced copies and the body runs unchanged - same statements, same
order, so results equal the oracle's bit for bit."""
import numpy as np
import pytest

import cases
from helpers import DRYRUN, assert_exact

pytestmark = pytest.mark.gpu


def _ops(ovl):
    @ovl.operator()
    def rowsum(a):
        out = ovl.output([a.shape[0]], a.dtype)
        row = ovl.position_in([a.shape[0]])[0]
        acc = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[1]):
            acc <<= acc + a[row, i]
        out[row] = acc
        return out

    @ovl.operator()
    def rowmax_and_last(a):
        # not a sum or a product: the running maximum, and a second output that reads the row outside the loop
        best = ovl.output([a.shape[0]], a.dtype)
        last = ovl.output([a.shape[0]], a.dtype)
        row = ovl.position_in([a.shape[0]])[0]
        m = ovl.variable(a[row, 0], a.dtype)
        for i in ovl.arange(1, a.shape[1]):
            m <<= ovl.maximum(m, a[row, i])
        best[row] = m
        last[row] = a[row, a.shape[1] - 1]
        return best, last
    return rowsum, rowmax_and_last


def _check(ns, outputs, monkeypatch=None):
    from opveclib_b200 import runtime
    from oracle import runner
    got = ns.ovl.evaluate(outputs, target_language='b200')
    prog, _ = runtime.compile_outputs(outputs)
    assert prog.plans[0].meta['rows'] is not None
    if DRYRUN:
        pytest.skip('compiled; needs a device to run')
    assert prog.plans[0].last_variant == 'rows'
    want = runner.evaluate(outputs)
    got = got if isinstance(got, list) else [got]
    want = want if isinstance(want, list) else [want]
    for g, w in zip(got, want):
        assert_exact(g, w)
    return got


@pytest.mark.parametrize('shape,dtype', [((20000, 32), np.float32), ((5000, 100), np.float32), ((70001, 8), np.float32),
                                         ((3000, 17), np.float64), ((4099, 64), np.int32), ((1000, 100), np.int16)])
def test_row_sums_keep_the_serial_order(shape, dtype):
    ns = cases.impl()
    rowsum, _ = _ops(ns.ovl)
    rs = np.random.RandomState(shape[1])
    x = (rs.randint(-100, 100, shape) if np.dtype(dtype).kind == 'i' else rs.normal(0, 1, shape)).astype(dtype)
    _check(ns, [rowsum(x)])


def test_running_maximum_and_a_read_outside_the_loop():
    ns = cases.impl()
    _, rowmax_and_last = _ops(ns.ovl)
    x = np.random.RandomState(2).normal(0, 1, (9000, 48)).astype(np.float32)
    best, last = rowmax_and_last(x)
    got = _check(ns, [best, last])
    assert np.array_equal(got[0], x.max(axis=1)) and np.array_equal(got[1], x[:, -1])


def test_short_matrix_vector_product_and_rank_two_workgroup():
    ns = cases.impl()
    u = cases.user_ops(ns)
    rs = np.random.RandomState(3)
    m = rs.normal(0, 1, (4096, 64)).astype(np.float32)
    v = rs.normal(0, 1, 64).astype(np.float32)
    _check(ns, [u.matvec(m, v)])                       # the matrix is staged, the vector is read as written
    x = rs.uniform(0.9, 1.1, (300, 5, 40)).astype(np.float32)
    s = rs.uniform(1, 2, 5).astype(np.float32)
    _check(ns, [u.rowprod_scaled(x, s)])               # workers [300, 5], rows of 40


def test_same_bits_without_staging(monkeypatch):
    ns = cases.impl()
    rowsum, _ = _ops(ns.ovl)
    x = np.random.RandomState(5).normal(0, 1, (8000, 24)).astype(np.float32)
    staged = _check(ns, [rowsum(x)])[0]
    monkeypatch.setenv('OVL_ROWS_MODE', 'off')
    plain = ns.ovl.evaluate([rowsum(x)], target_language='b200')
    assert np.array_equal(staged, plain)


def test_rows_that_are_written_are_collected_and_stored_as_one_piece():
    """``out[row, i] = a[row, i] / sum`` after a first loop that forms the sum, and an inclusive scan of short lines of
    odd length (serial arithmetic, as the oracle's): input AND output rows go through shared memory."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def normalise(a):
        out = ovl.output_like(a)
        row = ovl.position_in([a.shape[0]])[0]
        acc = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[1]):
            acc <<= acc + a[row, i]
        for i in ovl.arange(a.shape[1]):
            out[row, i] = a[row, i] / acc
        return out

    rs = np.random.RandomState(8)
    x = rs.uniform(0.5, 2, (9001, 50)).astype(np.float32)
    for op in (normalise(x), ns.cumsum(x, axis=1), ns.cumprod(rs.uniform(0.9, 1.1, (4000, 7)).astype(np.float64), axis=1)):
        prog, _ = runtime.compile_outputs([op])
        assert prog.plans[0].meta['rows']['staged_outputs'], prog.plans[0].meta['rows']
        _check(ns, [op])


def test_partly_written_rows_are_not_collected():
    from opveclib_b200 import runtime
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def every_other(a):
        out = ovl.output_like(a)
        row = ovl.position_in([a.shape[0]])[0]
        for i in ovl.arange(0, a.shape[1] - 1, 2):
            out[row, i] = a[row, i] + a[row, i + 1]
        return out

    @ovl.operator()
    def positive_only(a):
        out = ovl.output_like(a)
        row = ovl.position_in([a.shape[0]])[0]
        for i in ovl.arange(a.shape[1]):
            with ovl.if_(a[row, i] > 0):
                out[row, i] = a[row, i]
        return out

    x = np.random.RandomState(9).normal(0, 1, (3000, 41)).astype(np.float32)     # (a stepped loop from 0 to 40)
    for op in (every_other(x), positive_only(x)):
        prog, _ = runtime.compile_outputs([op])
        rows = prog.plans[0].meta['rows']
        assert rows is not None and rows['staged'] and not rows['staged_outputs']
