"""The packed body of the tolerance lowering (opveclib_b200/cuda_pack.py) executed on the HOST.

The generated ``_vec`` kernel is compiled by g++ against stand-in headers (tests/host_shim) and run with the launch
geometry emulated by loops, then compared with the CPU oracle's run of the same kernel: graphs of exact arithmetic
bit for bit (packed pairs, branches turned into selects or masks, hoisted vector loads and stores must not change a
value), graphs with transcendental functions within rtol 1e-5 (the stand-ins use the host's libm)."""
import numpy as np
import pytest

import cases
import fuzz_graphs
import host_kernel
from helpers import assert_close, assert_exact
from opveclib_b200 import cuda_emit, cuda_pack
from opveclib_b200.fuse import merge_op_dag
from opveclib_b200.opgraph import build_op_dag
from oracle import runner


def _compare(kernel, ins, exact, what):
    call, meta = host_kernel.run_vec(kernel, 'tolerance')
    assert meta['vec']['paired']
    got = call(ins)
    want, _ = runner.run_kernel(kernel, ins)
    for k, (g, w) in enumerate(zip(got, want)):
        if exact:
            assert_exact(g.view(np.uint32), w.view(np.uint32), '%s output %d' % (what, k))
        else:
            fin = np.isfinite(w)
            scale = float(np.abs(w[fin]).max())
            assert_close(g, w, rtol=1e-5, atol=1e-6 * scale, what='%s output %d' % (what, k))


def test_branch_shapes_that_need_masks():
    """Branches that assign several variables, nested chains, a chain without else and a store under a condition:
    none of them collapses into one nested select."""
    ns = cases.impl()
    ovl = ns.ovl

    @ovl.operator()
    def tangle(a, b):
        out = ovl.output_like(a)
        side = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        p = ovl.variable(0, a.dtype)
        q = ovl.variable(1, a.dtype)
        with ovl.if_(a[pos] > b[pos]):
            p <<= a[pos] - b[pos]
            q <<= a[pos] * 2.0
            with ovl.if_(a[pos] > 1.0):
                p <<= p + 0.25
            with ovl.elif_(b[pos] < -1.0):
                q <<= q - b[pos]
        with ovl.elif_(a[pos] < -0.5):
            p <<= b[pos] * b[pos]
        with ovl.if_(ovl.logical_or(p > 2.0, q < 0.0)):
            side[pos] = p * q
        with ovl.else_():
            side[pos] = ovl.minimum(p, q) - ovl.maximum(a[pos], b[pos])
        out[pos] = p + q * 0.5
        return out, side

    rs = np.random.RandomState(4)
    a = rs.uniform(-2, 2, (3, 1024)).astype(np.float32)
    b = rs.uniform(-2, 2, (3, 1024)).astype(np.float32)
    op = tangle(a, b)
    kernel = build_op_dag(op[0], op[1]).kernels[0]
    _compare(kernel, [a, b], True, 'tangle')


@pytest.mark.parametrize('name', ['chain16_light', 'chain16', 'c1_chain', 'lstm_fwd', 'lstm_grad', 'stdops_lstm'])
def test_benchmark_graphs_through_the_packed_body(name):
    ns = cases.impl()
    outs, _ = cases.CASES[name](ns)
    dag = merge_op_dag(build_op_dag(*outs))
    assert len(dag.kernels) == 1
    ins = [np.asarray(dag.inputs[ref.dag_input_index]) for ref in dag.references[0]]
    _compare(dag.kernels[0], ins, name == 'chain16_light', name)


@pytest.mark.parametrize('seed', range(40))
def test_random_exact_graphs_through_the_packed_body(seed):
    """Every kernel of the random graphs (fused) that qualifies for pairing gives, on the host, the bits the oracle
    gives for that kernel."""
    ns = cases.impl()
    outs, _ = fuzz_graphs.build(ns, seed)
    fused = merge_op_dag(build_op_dag(*outs))
    ran = 0
    for op_index, kernel in enumerate(fused.kernels):
        plan = cuda_emit.plan_vectorisation(kernel)
        if not plan.usable or cuda_pack.plan_pairs(kernel, plan) is None:
            continue
        rs = np.random.RandomState(1000 + seed * 17 + op_index)
        assert all(t.dtype.name == 'float32' for t in kernel.input_types + kernel.output_types)
        ins = [rs.uniform(-2, 2, t.shape).astype(np.float32) for t in kernel.input_types]
        _compare(kernel, ins, True, 'seed %d kernel %d' % (seed, op_index))
        ran += 1
    if ran == 0:
        pytest.skip('no kernel of this graph qualifies for pairing')


def test_only_fp32_bodies_are_paired():
    """Data movement and arithmetic in any other type keeps the scalar body: a pair holds two floats."""
    ns = cases.impl()
    seen = 0
    for seed in range(40):
        outs, _ = fuzz_graphs.build(ns, seed)
        for kernel in merge_op_dag(build_op_dag(*outs)).kernels:
            if all(t.dtype.name == 'float32' for t in kernel.input_types + kernel.output_types):
                continue
            plan = cuda_emit.plan_vectorisation(kernel)
            assert not plan.usable or cuda_pack.plan_pairs(kernel, plan) is None
            seen += 1
    assert seen > 10


@pytest.mark.parametrize('seed', range(40))
def test_vectorised_kernels_of_random_graphs_on_the_host(seed):
    """The exact lowering's vectorised kernels (hoisted 128-bit loads and stores, uniform loads, widened conditional
    stores) of the random graphs, any dtype, against the oracle's run of the same kernel."""
    ns = cases.impl()
    outs, _ = fuzz_graphs.build(ns, seed)
    ran = 0
    for op_index, kernel in enumerate(merge_op_dag(build_op_dag(*outs)).kernels):
        if not cuda_emit.plan_vectorisation(kernel).usable:
            continue
        rs = np.random.RandomState(7000 + seed * 13 + op_index)
        ins = []
        for t in kernel.input_types:
            if t.dtype.is_float:
                ins.append(rs.uniform(-2, 2, t.shape).astype(t.dtype.as_numpy()))
            else:
                lo = 0 if t.dtype.name.startswith('u') else -3
                ins.append(rs.randint(lo, 4, t.shape).astype(t.dtype.as_numpy()))
        call, _ = host_kernel.run_vec(kernel, 'exact')
        got = call(ins)
        want, _ = runner.run_kernel(kernel, ins)
        for k, (g, w) in enumerate(zip(got, want)):
            assert_exact(g.view(np.uint8), w.view(np.uint8), 'seed %d kernel %d output %d' % (seed, op_index, k))
        ran += 1
    if ran == 0:
        pytest.skip('no kernel of this graph has a vectorised variant')
