"""Recognition of the per-worker reduction loop (opveclib_b200/patterns.py): what is accepted and, more
important, what is left to the generic kernel."""
import numpy as np

import cases
from opveclib_b200 import patterns
from opveclib_b200.opgraph import build_op_dag


def _kernel(op):
    return build_op_dag(op).kernels[0]


def _spec(op):
    return patterns.match_reduce(_kernel(op))


def test_reference_reductions_are_recognised():
    ns = cases.impl()
    u = cases.user_ops(ns)
    spec = _spec(u.dot(np.zeros((4, 1000)), np.zeros((4, 1000))))
    assert spec is not None and spec.op == 'add' and spec.n == 1000
    spec = _spec(u.matvec(np.zeros((4, 300), np.float32), np.zeros(300, np.float32)))
    assert spec is not None and spec.op == 'add' and spec.n == 300
    spec = _spec(u.rowprod_scaled(np.zeros((2, 3, 500), np.float32), np.zeros(3, np.float32)))
    assert spec is not None and spec.op == 'mul' and spec.n == 500


def test_short_loops_and_scans_stay_generic():
    ns = cases.impl()
    u = cases.user_ops(ns)
    assert _spec(u.dot(np.zeros((100, 10)), np.zeros((100, 10)))) is None           # 10 iterations
    assert _spec(ns.cumsum(np.zeros((4, 2048), np.float32), axis=1)) is None          # writes inside the loop


def test_loops_with_other_effects_are_rejected():
    ovl = cases.impl().ovl
    x = np.zeros((4, 512), np.float32)

    @ovl.operator()
    def observed(a):
        # the running value is read inside the loop by something other than the update
        out = ovl.output(a.shape[0], a.dtype)
        pos = ovl.position_in(a.shape[0])[0]
        acc = ovl.variable(0, a.dtype)
        peak = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[1]):
            acc <<= acc + a[pos, i]
            peak <<= ovl.maximum(peak, acc)
        out[pos] = peak
        return out

    @ovl.operator()
    def conditional(a):
        out = ovl.output(a.shape[0], a.dtype)
        pos = ovl.position_in(a.shape[0])[0]
        acc = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[1]):
            with ovl.if_(a[pos, i] > 0):
                acc <<= acc + a[pos, i]
        out[pos] = acc
        return out

    @ovl.operator()
    def self_term(a):
        # the folded-in term depends on the accumulator itself
        out = ovl.output(a.shape[0], a.dtype)
        pos = ovl.position_in(a.shape[0])[0]
        acc = ovl.variable(1, a.dtype)
        for i in ovl.arange(a.shape[1]):
            acc <<= acc + acc * a[pos, i]
        out[pos] = acc
        return out

    @ovl.operator()
    def offset_start(a):
        out = ovl.output(a.shape[0], a.dtype)
        pos = ovl.position_in(a.shape[0])[0]
        acc = ovl.variable(0, a.dtype)
        for i in ovl.arange(1, a.shape[1]):
            acc <<= acc + a[pos, i]
        out[pos] = acc
        return out

    @ovl.operator()
    def subtracting(a):
        out = ovl.output(a.shape[0], a.dtype)
        pos = ovl.position_in(a.shape[0])[0]
        acc = ovl.variable(0, a.dtype)
        for i in ovl.arange(a.shape[1]):
            acc <<= acc - a[pos, i]
        out[pos] = acc
        return out

    for op in (observed, conditional, self_term, offset_start, subtracting):
        assert _spec(op(x)) is None, op


def test_unassigned_variable_gives_the_trip_count():
    """``arange(variable(shape[1], uint32))`` - the reference's dot - has a constant trip count."""
    from opveclib_b200.access import analyze
    u = cases.user_ops(cases.impl())
    k = _kernel(u.dot(np.zeros((4, 777)), np.zeros((4, 777))))
    info = analyze(k)
    assert list(info.loop_vars.values()) == [('l', 0)] and info.ranges[('l', 0)] == (0, 776)


def test_scans_along_any_axis_are_recognised_with_their_geometry():
    ns = cases.impl()
    for shape, axis, want in [((4, 2048), 1, (4, 2048, 4, 1)), ((4096, 64), 0, (64, 4096, 1, 64)),
                              ((3, 500, 7), 1, (21, 500, 3, 7)), ((5000,), 0, (1, 5000, 1, 1)),
                              ((2, 3, 4, 300), 2, (1800, 4, 6, 300))]:
        spec = patterns.match_scan(_kernel(ns.cumsum(np.zeros(shape, np.float32), axis=axis)))
        assert spec is not None and (spec.lines, spec.n, spec.outer, spec.inner) == want, (shape, axis)
