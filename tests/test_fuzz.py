"""Random operator graphs (tests/fuzz_graphs.py): fusion must not change a bit on the CPU oracle, and the CUDA path -
generic, vectorised, fused or not - must reproduce the oracle exactly (the graphs use only exactly rounded
arithmetic, comparisons and data movement)."""
import os

import numpy as np
import pytest

import cases
import fuzz_graphs
from helpers import DRYRUN, assert_exact

# OVL_FUZZ_SEEDS=first:last runs another range of seeds
_first, _last = (int(v) for v in os.environ.get('OVL_FUZZ_SEEDS', '0:40').split(':'))
SEEDS = list(range(_first, _last))


@pytest.mark.parametrize('seed', SEEDS)
def test_fusion_keeps_every_bit_on_the_oracle(seed):
    from opveclib_b200.fuse import merge_op_dag
    from opveclib_b200.opgraph import build_op_dag
    from oracle import runner
    outs, _ = fuzz_graphs.build(cases.impl(), seed)
    dag = build_op_dag(*outs)
    fused = merge_op_dag(dag)
    assert len(fused.kernels) <= len(dag.kernels)
    plain, _ = runner.run_dag(dag)
    merged, _ = runner.run_dag(fused)
    for i, (a, b) in enumerate(zip(plain, merged)):
        assert_exact(b, a, 'seed %d output %d' % (seed, i))


@pytest.mark.gpu
@pytest.mark.parametrize('opt_level', [0, 3])
@pytest.mark.parametrize('seed', SEEDS)
def test_cuda_reproduces_the_oracle_exactly(seed, opt_level):
    from oracle import runner
    ns = cases.impl()
    outs, _ = fuzz_graphs.build(ns, seed)
    got = ns.ovl.evaluate(outs, opt_level=opt_level)
    if DRYRUN:
        return
    want = runner.evaluate(outs)
    if len(outs) == 1:
        got, want = [got], [want]
    for i, (g, w) in enumerate(zip(got, want)):
        assert_exact(np.asarray(g), w, 'seed %d opt %d output %d' % (seed, opt_level, i))


@pytest.mark.gpu
@pytest.mark.parametrize('seed', SEEDS)
def test_tolerance_lowering_keeps_exact_arithmetic_exact(seed):
    """The graphs use no division and no transcendental function, so the tolerance lowering may change nothing: its
    packed two-element additions, subtractions and multiplications round like single ones, and conditionals turned
    into selects pick the same values.  (Bodies of pure fp32 arithmetic take the packed path; everything else runs
    the same code in both lowerings.)"""
    from oracle import runner
    ns = cases.impl()
    outs, _ = fuzz_graphs.build(ns, seed)
    got = ns.ovl.evaluate(outs, math='tolerance')
    if DRYRUN:
        return
    want = runner.evaluate(outs)
    if len(outs) == 1:
        got, want = [got], [want]
    for i, (g, w) in enumerate(zip(got, want)):
        assert_exact(np.asarray(g), w, 'seed %d output %d (tolerance lowering)' % (seed, i))
