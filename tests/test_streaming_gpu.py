"""Row-streamed evaluation of host-resident graphs gives exactly what the one-piece evaluation gives."""
import numpy as np
import pytest

import cases
from helpers import DRYRUN, assert_exact

pytestmark = pytest.mark.gpu


def _both_ways(build, host_inputs):
    """Evaluate once from host arrays (streamed when the graph allows it) and once from device tensors."""
    import torch
    from opveclib_b200 import runtime, streaming
    ns = cases.impl()
    outs = build(ns, *host_inputs)
    prog, dag = runtime.compile_outputs(outs)
    plan = streaming.plan(outs, dag, prog, 3)
    streamed = ns.ovl.evaluate(outs)
    if DRYRUN:
        return plan, None, None
    dev_outs = build(ns, *[torch.from_numpy(a).cuda() for a in host_inputs])
    whole = ns.ovl.evaluate(dev_outs)
    if not isinstance(streamed, list):
        streamed, whole = [streamed], [whole]
    return plan, streamed, [w.cpu().numpy() for w in whole]


def test_fused_chain_is_streamed_in_fine_slabs():
    """An element-local graph over few long rows is viewed as more, shorter rows (same memory) so that the slabs
    that travel alone at the start and at the end are small."""
    x = np.random.RandomState(0).uniform(-2, 2, (8, 1 << 21)).astype(np.float32)
    plan, streamed, whole = _both_ways(lambda ns, a: [cases.chain16(ns, a)], [x])
    assert plan is not None and plan['slabs'] == 32 and plan['slab_rows'] == 1 and plan['view'] == [32, 1 << 19]
    if streamed is not None:
        assert_exact(streamed[0], whole[0], 'streamed chain16')


def test_odd_extents_fall_back_to_slabs_of_rows():
    x = np.random.RandomState(2).uniform(-2, 2, (6, (1 << 21) + 4)).astype(np.float32)
    plan, streamed, whole = _both_ways(lambda ns, a: [cases.chain16_light(ns, a)], [x])
    assert plan is not None and plan['slabs'] * plan['slab_rows'] == plan['rows']
    if streamed is not None:
        assert_exact(streamed[0], whole[0], 'streamed light chain')


def test_lstm_cell_is_streamed_over_the_batch():
    rs = np.random.RandomState(1)
    g = rs.normal(0, 1, (96, 4 * 32768)).astype(np.float32)
    c = rs.normal(0, 1, (96, 32768)).astype(np.float32)

    def build(ns, gates, cell):
        op = ns.lstm(gates, cell, forget_bias=0.0)
        return [op[0], op[1]]
    plan, streamed, whole = _both_ways(build, [g, c])
    assert plan is not None and plan['slabs'] == 8 and plan['slab_rows'] == 12
    if streamed is not None:
        for s, w in zip(streamed, whole):
            assert_exact(s, w, 'streamed lstm')
    # results can be written into caller-provided (e.g. pinned) arrays
    if streamed is not None:
        ns = cases.impl()
        out = [np.empty_like(streamed[0]), np.empty_like(streamed[1])]
        got = ns.ovl.evaluate(build(ns, g, c), out=out)
        assert got[0] is out[0] and np.array_equal(out[1], whole[1])


def test_graphs_that_are_not_row_local_are_evaluated_in_one_piece():
    from opveclib_b200 import runtime, streaming
    ns = cases.impl()
    for outs in ([ns.cumsum(np.zeros((64, 1 << 18), np.float32), axis=1)],             # loop along the row
                 [cases.user_ops(ns).shift_cyclic(np.zeros(1 << 24, np.float32))],    # rows exchange elements
                 [ns.cumsum(np.zeros((1 << 12, 4096), np.float32), axis=0)]):          # scan down the rows
        prog, dag = runtime.compile_outputs(outs)
        assert streaming.plan(outs, dag, prog, 3) is None


def test_shape_derived_constants_keep_the_graph_in_one_piece():
    """An operator that bakes a number taken from its input's shape into a value computes something else when it is
    traced again for a slab; such graphs are not streamed, and the result is the one-piece result."""
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def mean_scaled(x):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = x[pos] / float(x.shape[0]) + float(x.shape[1])
        return out

    x = np.random.RandomState(3).uniform(-1, 1, (16, 1 << 20)).astype(np.float32)

    def build(ns_, a):
        return [mean_scaled(a)]
    plan, streamed, whole = _both_ways(build, [x])
    assert plan is None
    if streamed is not None:
        assert_exact(streamed[0], whole[0], 'shape-derived constants')
        assert_exact(streamed[0], x / np.float32(16.0) + np.float32(1 << 20), 'value')
