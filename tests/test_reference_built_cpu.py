"""The reference-built CPU operators (oracle/_ref: C++ that the reference's own tracer, merger and generator
emitted, compiled against its headers) and this repository's oracle port must agree bit for bit on the benchmark
workloads.  Skipped where oracle/_ref has not been built."""
import numpy as np
import pytest

import cases
from helpers import assert_exact
from oracle import ref_runner, runner

pytestmark = pytest.mark.skipif(not ref_runner.available(), reason='oracle/_ref has not been built')


def _inputs(name):
    rs = np.random.RandomState(77)
    f32 = np.float32
    if name == 'c1_chain_1048576' or name == 'c1_shift_1048576':
        return [rs.uniform(-1, 1, 1 << 20).astype(f32)]
    if name == 'c2_cumsum_4096x8192':
        return [rs.normal(0, 1, (4096, 8192)).astype(f32)]
    if name == 'c2_cumprod_4096x8192':
        return [rs.uniform(0.99, 1.01, (4096, 8192)).astype(f32)]
    if name == 'c3_lstm_512x1024':
        return [rs.normal(0, 1, (512, 4096)).astype(f32), rs.normal(0, 1, (512, 1024)).astype(f32)]
    if name == 'c3_lstm_grad_512x1024':
        return [rs.normal(0, 1, (512, 4096)).astype(f32), rs.normal(0, 1, (512, 1024)).astype(f32),
                rs.normal(0, 0.1, (512, 1024)).astype(f32), rs.normal(0, 0.1, (512, 1024)).astype(f32)]
    if name == 'c4_chain16_1x16777216':
        return [rs.uniform(-2, 2, (1, 1 << 24)).astype(f32)]
    raise KeyError(name)


def _port(name, ins):
    ns = cases.impl()
    u = cases.user_ops(ns)
    if name == 'c1_chain_1048576':
        return [cases.c1_chain(ns, ins[0])]
    if name == 'c1_shift_1048576':
        return [u.shift_cyclic(ins[0])]
    if name == 'c2_cumsum_4096x8192':
        return [ns.cumsum(ins[0], axis=1)]
    if name == 'c2_cumprod_4096x8192':
        return [ns.cumprod(ins[0], axis=1)]
    if name == 'c3_lstm_512x1024':
        op = ns.lstm(ins[0], ins[1], forget_bias=0.0)
        return [op[0], op[1]]
    if name == 'c3_lstm_grad_512x1024':
        op = ns.lstm_grad(ins[0], ins[1], ins[2], ins[3], forget_bias=0.0)
        return [op[0], op[1]]
    if name == 'c4_chain16_1x16777216':
        return [cases.chain16(ns, ins[0])]
    raise KeyError(name)


@pytest.mark.parametrize('name', ['c1_chain_1048576', 'c1_shift_1048576', 'c2_cumsum_4096x8192', 'c2_cumprod_4096x8192',
                                  'c3_lstm_512x1024', 'c3_lstm_grad_512x1024', 'c4_chain16_1x16777216'])
def test_reference_built_operators_equal_the_oracle_port(name):
    if not ref_runner.available(name):
        pytest.skip(name + ' is not in oracle/_ref')
    ins = _inputs(name)
    ref_outs, _ = ref_runner.run(name, ins, num_threads=0, variant='opt', iterations=1)
    outs = _port(name, ins)
    want = runner.evaluate(outs)
    if len(outs) == 1:
        want = [want]
    assert len(ref_outs) == len(want)
    for k, (a, b) in enumerate(zip(ref_outs, want)):
        assert_exact(np.asarray(a).reshape(b.shape), b, '%s output %d: reference-built vs port' % (name, k))


def test_reference_flags_and_optimised_build_agree():
    """The reference compiles its operators without optimisation; the -O2 -ffp-contract=off build that serves as
    CPU baseline computes the same bits."""
    name = 'c3_lstm_512x1024'
    if not ref_runner.available(name):
        pytest.skip(name + ' is not in oracle/_ref')
    ins = _inputs(name)
    a, _ = ref_runner.run(name, ins, num_threads=0, variant='opt', iterations=1)
    b, _ = ref_runner.run(name, ins, num_threads=0, variant='ref', iterations=1)
    for x, y in zip(a, b):
        assert_exact(x, y, 'reference flags vs -O2')
