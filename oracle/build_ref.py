"""TEST INFRASTRUCTURE - never part of the product path.

Builds ``oracle/_ref``: the REFERENCE's own CPU implementation of the benchmark workloads, compiled from what
the reference generates, so that it can be timed (and used as a checker) on a machine where the reference tree
and its Python dependencies are absent.

    python oracle/build_ref.py            # needs the reference tree (development container only)

For every workload below the reference package (loaded through oracle/ref_shim.py) traces the operators, builds
and merges the operator graph exactly as its ``profile`` does (opveclib/operator.py:2256-2259), and emits the C++
source of every operator with ``ExpressionDAG.generate`` (opveclib/expression.py:522-706).  Each source is
compiled twice against the reference's ``dynamiclibop.h`` where it lies: with the reference's flags (no
optimisation, opveclib/operator.py:2051-2055) and with ``-O2 -ffp-contract=off`` (bit-identical results, no
contraction).  ``manifest.json`` records, per workload, the operators in execution order, their wiring and
types.  Outputs go only to ``oracle/_ref`` (git-ignored); nothing from the reference is copied into the
repository.  ``oracle/ref_runner.py`` executes a manifest entry on numpy arrays.
"""
import json
import os
import subprocess
import sys
import tempfile
import warnings

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, '_ref')
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'tests'))

# workload name -> builder(ns) returning the operator outputs; inputs are placeholders of the right type only
C4_SAMPLE_COLS = 1 << 24
C5_SAMPLE = 1 << 26


def workloads(ns):
    import cases
    f32 = np.float32
    z = lambda *shape: np.zeros(shape, dtype=f32)
    u = cases.user_ops(ns)
    lstm = ns.lstm(z(512, 4096), z(512, 1024), forget_bias=0.0)
    lstm_grad = ns.lstm_grad(z(512, 4096), z(512, 1024), z(512, 1024), z(512, 1024), forget_bias=0.0)
    return {
        'c1_chain_1048576': [cases.c1_chain(ns, z(1 << 20))],
        'c1_shift_1048576': [u.shift_cyclic(z(1 << 20))],
        'c2_cumsum_4096x8192': [ns.cumsum(z(4096, 8192), axis=1)],
        'c2_cumprod_4096x8192': [ns.cumprod(z(4096, 8192), axis=1)],
        'c3_lstm_512x1024': [lstm[0], lstm[1]],
        'c3_lstm_grad_512x1024': [lstm_grad[0], lstm_grad[1]],
        'c4_chain16_1x%d' % C4_SAMPLE_COLS: [cases.chain16(ns, z(1, C4_SAMPLE_COLS))],
        'c5_cumsum_%d' % C5_SAMPLE: [ns.cumsum(z(C5_SAMPLE))],
        # the same operator traced for fp64 input: "run in fp64 and cast", the oracle of the sharded scan
        'c5_cumsum_f64_%d' % C5_SAMPLE: [ns.cumsum(np.zeros(C5_SAMPLE, dtype=np.float64))],
    }


def main():
    warnings.simplefilter('ignore')
    from oracle import ref_shim
    if not ref_shim.available():
        print('reference tree not present: oracle/_ref not built')
        return 0
    os.makedirs(OUT, exist_ok=True)
    ns = ref_shim.load(tempfile.mkdtemp(prefix='ovl_ref_'))
    opmod = ns.opmod
    ref_shim.build_harness(os.path.join(OUT, 'libref_harness.so'))
    inc = '-I' + os.path.join(ref_shim.REFERENCE_ROOT, 'opveclib')
    cxx = os.getenv('OPVECLIB_CXX', 'g++')
    manifest = {}
    for name, outs in sorted(workloads(ns).items()):
        op_dag = opmod._build_op_dag(*outs)
        dag = op_dag.proto_dag
        opt_level = 3
        try:
            dag, _ = opmod._merge_op_dag(dag, None)
        except Exception as exc:      # the reference's merger raises on some graphs; fall back to no merging
            print('  %s: reference merge failed (%s: %s); using the unmerged graph' % (name, type(exc).__name__, exc))
            dag, opt_level = op_dag.proto_dag, 0
        entry = {'opt_level': opt_level, 'ops': [], 'outputs': [], 'inputs': []}
        for t in dag.dag_input_types:
            entry['inputs'].append([int(t.dtype), [int(d) for d in t.shape]])
        for op_index, op in enumerate(dag.operators):
            fname = opmod._op_hash(op)
            c_src, _ = opmod.ExpressionDAG.generate(op, fname)
            in_types, out_types = opmod.ExpressionDAG.io_types()
            src_path = os.path.join(OUT, fname + '_generic_cpp.cpp')
            with open(src_path, 'w') as f:
                f.write(c_src)
            for variant, flags in (('ref', ['-g']), ('opt', ['-O2', '-ffp-contract=off'])):
                so = os.path.join(OUT, fname + '_' + variant + '.so')
                if not os.path.exists(so):
                    subprocess.check_output([cxx, '-fPIC', '-std=c++11', '-w', inc, '-shared'] + flags +
                                            ['-o', so, src_path], stderr=subprocess.STDOUT)
            refs = []
            for r in dag.references[op_index].input_refs:
                refs.append(['L', int(r.dag_input_index)] if r.is_leaf else ['O', int(r.op_index), int(r.op_output_index)])
            entry['ops'].append({'name': op.name, 'lib': fname, 'fn': fname + '_generic_cpp', 'inputs': refs,
                                 'in_types': [[int(t.dtype.proto_dtype), list(t.shape)] for t in in_types],
                                 'out_types': [[int(t.dtype.proto_dtype), list(t.shape)] for t in out_types]})
        for o in dag.dag_outputs:
            entry['outputs'].append([int(o.op_index), int(o.op_output_index)])
        manifest[name] = entry
        print('%-28s %d operator(s) after the reference merge (opt_level %d)' % (name, len(entry['ops']), opt_level))
    with open(os.path.join(OUT, 'manifest.json'), 'w') as f:
        json.dump(manifest, f, indent=1)
    return 0


if __name__ == '__main__':
    sys.exit(main())
