"""The CPU oracle against golden vectors recorded from the reference implementation.

Each fixture holds the inputs and the outputs the reference's own generated C++ operators produced
(tests/golden/make_golden.py).  The oracle re-derives the operators from this package's tracer and its own
restatement of the reference's C++ generator; being the same arithmetic on the same libm it must reproduce the
reference bit for bit.  For transcendental cases one unit in the last place is tolerated so that a host whose
libm picks different code paths (FMA variants) does not fail the pin.
"""
import numpy as np
import pytest

import cases
from helpers import assert_exact, load_golden, ulp_diff
from oracle import runner


@pytest.mark.parametrize('name', sorted(cases.CASES))
def test_oracle_reproduces_reference(name):
    ins, want = load_golden(name)
    outs, case_ins = cases.CASES[name](cases.impl())
    for a, b in zip(case_ins, ins):
        assert_exact(np.asarray(a), b, name + ' input')
    got = runner.evaluate(outs)
    if len(outs) == 1:
        got = [got]
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        what = '%s output %d' % (name, i)
        if name in cases.TRANSCENDENTAL and g.dtype.kind == 'f':
            assert g.shape == w.shape and g.dtype == w.dtype
            fin = np.isfinite(w)
            assert np.array_equal(np.isfinite(g), fin), what
            assert ulp_diff(np.where(fin, g, 0), np.where(fin, w, 0)).max() <= 1, what
        else:
            assert_exact(g, w, what)


@pytest.mark.parametrize('name', ['c1_chain', 'chain16', 'stdops_lstm', 'merge_graph', 'lstm_grad', 'merge_scan_nested',
                                  'merge_scan_rows_then_cols', 'merge_product_then_scan', 'merge_pad_crop',
                                  'merge_add_tree', 'merge_product_split_adds'])
def test_fused_graph_equals_unfused_on_cpu(name):
    """Fusion must not change a single bit: the fused graph run through the oracle equals the unfused one."""
    from opveclib_b200.fuse import merge_op_dag
    from opveclib_b200.opgraph import build_op_dag
    outs, _ = cases.CASES[name](cases.impl())
    dag = build_op_dag(*outs)
    fused = merge_op_dag(dag)
    a, _ = runner.run_dag(dag)
    b, _ = runner.run_dag(fused)
    assert len(fused.kernels) <= len(dag.kernels)
    for i, (x, y) in enumerate(zip(a, b)):
        assert_exact(y, x, '%s output %d' % (name, i))
