"""Record golden vectors by running the REFERENCE implementation on the shared test cases.

Run in the development container, where the reference tree is mounted:

    python tests/golden/make_golden.py

For every case of tests/cases.py the operators are built with the reference package (through
oracle/ref_shim.py, which adapts the unmodified reference to this container) and evaluated by the reference's
own ``evaluate(..., target_language='cpp')``: its tracer, its merge optimizer, its C++ generator, g++ with the
reference's flags, and its generated operator code run on host threads.  Inputs and outputs are stored as
``tests/golden/<case>.npz`` (``in_<i>``, ``out_<i>``).  The fixtures pin the CPU oracle of this repository
(tests/test_oracle_golden.py) and, with tolerances, the CUDA path (tests/test_parity_gpu.py).
"""
import os
import sys
import tempfile
import warnings

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'tests'))


def main(argv):
    warnings.simplefilter('ignore')
    from oracle import ref_shim
    ns = ref_shim.load(tempfile.mkdtemp(prefix='ovl_ref_'))
    import cases
    wanted = argv[1:] or sorted(cases.CASES)
    for name in wanted:
        outs, ins = cases.CASES[name](ns)
        try:
            res = ns.ovl.evaluate(outs, target_language='cpp', opt_level=3)
            if len(outs) == 1:
                res = [res]
        except Exception as exc:   # the reference's merge optimizer raises on some graphs
            print('  note: reference opt_level=3 evaluation of %s raised %s: %s' % (name, type(exc).__name__, exc))
            res = None
        unmerged = ns.ovl.evaluate(outs, target_language='cpp', opt_level=0)
        if len(outs) == 1:
            unmerged = [unmerged]
        if res is None:
            try:
                res = [ns.ovl.evaluate([o], target_language='cpp', opt_level=3) for o in outs]
            except Exception:
                print('  note: per-output opt_level=3 evaluation raised too; recording opt_level=0 results')
                res = unmerged
        if not all(np.array_equal(a, b, equal_nan=True) for a, b in zip(res, unmerged)):
            # Seen for graphs of several independent operators evaluated in one call: the reference's merged
            # graph then runs some operators with another operator's workgroup and leaves 0xFE fill behind.
            # Each output evaluated on its own (still opt_level=3) is correct; record those.
            print('  note: reference opt_level=3 joint evaluation of %s disagrees with opt_level=0; '
                  'recording per-output evaluations' % name)
            res = [ns.ovl.evaluate([o], target_language='cpp', opt_level=3) for o in outs]
            if not all(np.array_equal(a, b, equal_nan=True) for a, b in zip(res, unmerged)):
                # Seen for a scan fed by another scan of the same workgroup (the reference merges them through a
                # temporary buffer, opveclib/test/test_operator_merge.py:227-236, and the merged operator computes
                # something else).  The unmerged evaluation is the operators' meaning; record that.
                print('  note: reference opt_level=3 evaluation of %s disagrees with opt_level=0 even per output; '
                      'recording the opt_level=0 results' % name)
                res = unmerged
        payload = {}
        for i, a in enumerate(ins):
            payload['in_%d' % i] = np.asarray(a)
        for i, a in enumerate(res):
            payload['out_%d' % i] = np.asarray(a)
        np.savez_compressed(os.path.join(HERE, name + '.npz'), **payload)
        print('%-24s %d inputs %d outputs' % (name, len(ins), len(res)))


if __name__ == '__main__':
    main(sys.argv)
