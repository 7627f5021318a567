"""Record golden vectors for the triangle-counting example by running the REFERENCE's own code.

Run in the development container, where the reference tree is mounted:

    python tests/golden/make_golden_graph.py

The reference's edge-list loader, its plain-Python counter and its ``triangles_op`` operator (evaluated by the
reference's own ``evaluate(..., target_language='cpp')`` through oracle/ref_shim.py) are run on two edge lists: the
example graph the reference's test writes (7 vertices, 20 directed edges, 3 triangles) and a seeded random list with
gaps in the vertex ids, self-loops and repeated edges.  Stored in ``tests/golden/graph_<name>.npz``: the pairs as
read, the loader's three arrays, the per-edge counts of the operator and the total of the Python counter.
"""
import os
import sys
import tempfile
import warnings

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def random_pairs():
    rs = np.random.RandomState(20)
    ids = rs.choice(400, size=120, replace=False)           # vertex ids with gaps
    pairs = ids[rs.randint(0, 120, size=(1500, 2))]
    pairs[::50, 1] = pairs[::50, 0]                         # self-loops
    pairs[1::70] = pairs[0::70][:len(pairs[1::70]), ::-1]   # repeated edges, reversed
    return pairs.astype(np.uint64)


def main():
    warnings.simplefilter('ignore')
    from oracle import ref_shim
    work = tempfile.mkdtemp(prefix='ovl_ref_graph_')
    ns = ref_shim.load(work)
    import opveclib.examples.test_graph as ref_graph
    cases = {}
    example = os.path.join(work, 'example.txt')
    ref_graph.write_example_graph_to_text_file(example)
    cases['example'] = np.loadtxt(example, dtype=np.uint64).reshape(-1, 2)
    cases['random'] = random_pairs()
    for name, pairs in cases.items():
        path = os.path.join(work, name + '.txt')
        with open(path, 'w') as f:
            for a, b in pairs:
                f.write('%d\t%d\n' % (a, b))
        start, frm, to = ref_graph.load_graph_from_text_file(path)
        per_edge = ns.ovl.evaluate(ref_graph.triangles_op(start, frm, to), target_language='cpp')
        total = ref_graph.reference(start, frm, to)
        assert int(np.sum(per_edge, dtype=np.uint64)) == total
        np.savez(os.path.join(HERE, 'graph_' + name + '.npz'), pairs=pairs, start=start, from_vertex=frm, to_vertex=to,
                 per_edge=per_edge, total=np.uint64(total))
        print('graph_%s: %d pairs -> %d edges, %d triangles' % (name, len(pairs), len(to), total))


if __name__ == '__main__':
    main()
