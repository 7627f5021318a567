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


# ---------------------------------------------------------------------------------------------------------
# accesses staged through shared memory (cuda_emit.plan_tiling) and the launch shape of the warp-per-line scan

def _tiling(op):
    from opveclib_b200 import cuda_emit
    from opveclib_b200.access import analyze
    k = _kernel(op)
    return cuda_emit.plan_tiling(k, analyze(k))


def test_transposed_operands_and_results_are_staged():
    ns = cases.impl()
    u = cases.user_ops(ns)
    axis, reads, writes, tile_t, tile_l = _tiling(u.transpose(np.zeros((200, 300), np.float32)))
    assert axis == 0 and len(reads) == 1 and not writes and (tile_t, tile_l) == (64, 64)
    axis, reads, writes, tile_t, tile_l = _tiling(u.transpose_axpy(np.zeros((40, 100), np.float32),
                                                                  np.zeros((100, 40), np.float32), alpha=1.0))
    assert axis == 0 and len(reads) == 1 and (tile_t, tile_l) == (64, 32)
    ovl = ns.ovl

    @ovl.operator()
    def scatter(a):
        out = ovl.output([a.shape[1], a.shape[0]], a.dtype)
        pos = ovl.position_in(a.shape)
        out[pos[1], pos[0]] = a[pos]
        return out

    axis, reads, writes, _, _ = _tiling(scatter(np.zeros((64, 96), np.float64)))
    assert axis == 0 and not reads and len(writes) == 1


def test_what_is_not_staged():
    ns = cases.impl()
    u = cases.user_ops(ns)
    ovl = ns.ovl
    assert _tiling(u.transpose(np.zeros((8, 300), np.float32))) is None        # the result is only 8 wide
    assert _tiling(u.ew_mulc(np.zeros((64, 64), np.float32), c=2.0)) is None    # nothing strided
    assert _tiling(u.shift_cyclic(np.zeros(4096, np.float32))) is None          # rank 1

    @ovl.operator()
    def guarded(a):
        # the transposed read sits behind a condition on a straight read: staged (the address is valid for every
        # worker); the conditional transposed write is not
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        with ovl.if_(a[pos] > 0):
            out[pos[1], pos[0]] = a[pos[1], pos[0]]
        return out

    axis, reads, writes, _, _ = _tiling(guarded(np.zeros((64, 64), np.float32)))
    assert len(reads) == 1 and not writes

    @ovl.operator()
    def strided_gather(a):
        # stride 2 along the innermost axis, no axis along which the operand is contiguous
        out = ovl.output([a.shape[0], a.shape[1] // 2], a.dtype)
        pos = ovl.position_in(out.shape)
        out[pos] = a[pos[0], pos[1] * 2]
        return out

    assert _tiling(strided_gather(np.zeros((64, 128), np.float32))) is None


def test_warp_scan_shape_divides_the_lines_evenly():
    from opveclib_b200 import runtime
    for lines in (2048, 4096, 5000, 20000, 32767):
        grid, block = runtime.warp_scan_shape(lines, 148)
        warps = block // 32
        assert 4 <= warps <= 8 and block % 32 == 0 and 1 <= grid <= 148 * 4
        slots = grid * warps
        rounds = -(-lines // slots)
        assert lines / float(rounds * slots) > 0.85
    assert runtime.warp_scan_shape(4096, 148) == (296, 224)      # two even rounds of 2072 warps
    # tens of thousands of lines: one line per warp, four warps per block
    assert runtime.warp_scan_shape(2 ** 17, 148) == (2 ** 15, 128)
    assert runtime.warp_scan_shape(10 ** 5 + 1, 148) == (25001, 128)


def test_reduction_layout_follows_the_contiguous_direction():
    """Column sums put neighbouring workers, not neighbouring trips, on the threads of a warp."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    u = cases.user_ops(ns)
    prog, _ = runtime.compile_outputs([u.colsum(np.zeros((300, 512), np.float32))])
    assert prog.plans[0].meta['red']['layout'] == 'across' and prog.plans[0].meta['red']['workers_per_block'] == 32
    prog, _ = runtime.compile_outputs([u.matvec(np.zeros((64, 300), np.float32), np.zeros(300, np.float32))])
    assert prog.plans[0].meta['red']['layout'] == 'along'
    prog, _ = runtime.compile_outputs([u.colsum(np.zeros((300, 16), np.float32))])      # half a warp of columns
    assert prog.plans[0].meta['red']['layout'] == 'across'
    prog, _ = runtime.compile_outputs([u.colsum(np.zeros((300, 4), np.float32))])       # too few columns for a warp
    assert prog.plans[0].meta['red']['layout'] == 'along'


def test_long_reduction_loops_of_few_workers_are_split_over_blocks():
    """One dot product of a million terms must not run on one SM: its loop is cut into slices for many blocks, the
    partial results meet in scratch memory behind the status header."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    u = cases.user_ops(ns)
    prog, _ = runtime.compile_outputs([u.matvec(np.zeros((3, 1 << 20), np.float32), np.zeros(1 << 20, np.float32))])
    red = prog.plans[0].meta['red']
    assert red['layout'] == 'along' and red['split']['units'] == 3 and red['split']['max'] == 64
    assert red['split']['zero_bytes'] == 32 and red['split']['scratch_bytes'] == 32 + 3 * 64 * 4
    prog, _ = runtime.compile_outputs([u.colsum(np.zeros((1 << 17, 48), np.float32))])
    red = prog.plans[0].meta['red']
    assert red['layout'] == 'across' and red['split']['units'] == 2 and red['block'] == 1024
    # many workers, or short loops: one block (or warp) per worker as before
    prog, _ = runtime.compile_outputs([u.matvec(np.zeros((4096, 1 << 16), np.float32), np.zeros(1 << 16, np.float32))])
    assert 'split' not in prog.plans[0].meta['red']
    prog, _ = runtime.compile_outputs([u.matvec(np.zeros((3, 4096), np.float32), np.zeros(4096, np.float32))])
    assert 'split' not in prog.plans[0].meta['red']


def test_seeded_scan_needs_assignment_before_the_first_store():
    """``acc <<= x[line, 0]; y[line, 0] = acc; for i in 1..n`` is an inclusive scan; with the first store in front
    of the assignment, y[line, 0] is the variable's initial value and the loop is left to the generic kernel."""
    ovl = cases.impl().ovl
    x = np.zeros((4, 4096), np.float32)

    def make(store_first):
        @ovl.operator()
        def scan(a):
            out = ovl.output_like(a)
            line = ovl.position_in([a.shape[0]])[0]
            acc = ovl.variable(0, a.dtype)
            if store_first:
                out[line, 0] = acc
                acc <<= a[line, 0]
            else:
                acc <<= a[line, 0]
                out[line, 0] = acc
            for i in ovl.arange(1, a.shape[1]):
                acc <<= acc + a[line, i]
                out[line, i] = acc
            return out
        return scan(x)

    assert patterns.match_scan(_kernel(make(False))) is not None
    assert patterns.match_scan(_kernel(make(True))) is None


def test_rows_read_in_a_loop_are_staged_and_others_are_not():
    """Row staging applies to inputs that a worker reads only inside its own row, with a read in a loop."""
    from opveclib_b200 import runtime
    ns = cases.impl()
    u = cases.user_ops(ns)
    prog, _ = runtime.compile_outputs([u.matvec(np.zeros((4096, 64), np.float32), np.zeros(64, np.float32))])
    assert prog.plans[0].meta['rows']['staged'] == [[0, 64]]            # the matrix, not the vector
    prog, _ = runtime.compile_outputs([u.matvec(np.zeros((4096, 8192), np.float32), np.zeros(8192, np.float32))])
    assert prog.plans[0].meta['rows'] is None                           # rows of 32 KB: the reduction kernel's
    prog, _ = runtime.compile_outputs([u.matvec(np.zeros((100, 64), np.float32), np.zeros(64, np.float32))])
    assert prog.plans[0].meta['rows'] is None                           # too few workers
    prog, _ = runtime.compile_outputs([u.colsum(np.zeros((64, 4096), np.float32))])
    assert prog.plans[0].meta['rows'] is None                           # a worker's reads are a column, not a row
    op = ns.lstm(np.zeros((512, 4096), np.float32), np.zeros((512, 1024), np.float32), forget_bias=0.0)
    prog, _ = runtime.compile_outputs([op[0], op[1]])
    assert prog.plans[0].meta['rows'] is None                           # no loop


def test_loop_nests_that_fold_into_one_accumulator():
    """A nest of two counted loops is one reduction over its trips; anything else in the outer body, or an inner
    loop whose length depends on the outer variable, leaves the kernel generic."""
    ovl = cases.impl().ovl
    x = np.zeros((4, 6, 20, 30), np.float32)

    def make(kind):
        @ovl.operator()
        def op(a):
            out = ovl.output([a.shape[0], a.shape[1]], a.dtype)
            pos = ovl.position_in([a.shape[0], a.shape[1]])
            acc = ovl.variable(0, a.dtype)
            rows = ovl.variable(0, a.dtype)
            for i in ovl.arange(a.shape[2]):
                if kind == 'effect':
                    rows <<= rows + 1
                for j in (ovl.arange(i + 1) if kind == 'triangle' else ovl.arange(a.shape[3])):
                    acc <<= acc + a[pos[0], pos[1], i, j]
            out[pos] = acc + rows
            return out
        return op

    spec = _spec(make('plain')(x))
    assert spec is not None and spec.n == 600 and spec.n_inner == 30 and spec.inner is not None
    assert _spec(make('effect')(x)) is None
    assert _spec(make('triangle')(x)) is None
