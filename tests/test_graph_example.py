"""The triangle-counting example (data-dependent indexing, a merge loop with a run-time trip count, nested
conditionals) against vectors recorded from the reference's own loader, operator and Python counter
(tests/golden/make_golden_graph.py; opveclib/examples/test_graph.py:371-401 is the reference's test)."""
import os

import numpy as np
import pytest

from helpers import DRYRUN, GOLDEN_DIR
from opveclib_b200.examples import graph


def _golden(name):
    return np.load(os.path.join(GOLDEN_DIR, 'graph_' + name + '.npz'))


@pytest.mark.parametrize('name', ['example', 'random'])
def test_loader_builds_the_reference_adjacency(name, tmp_path):
    g = _golden(name)
    start, frm, to = graph.adjacency_from_edges(g['pairs'])
    for got, want in ((start, g['start']), (frm, g['from_vertex']), (to, g['to_vertex'])):
        assert got.dtype == want.dtype and np.array_equal(got, want)
    path = str(tmp_path / 'edges.txt')
    with open(path, 'w') as f:
        f.write('# a comment line\n')
        for a, b in g['pairs']:
            f.write('%d\t%d\n' % (a, b))
    again = graph.load_graph_from_text_file(path)
    assert all(np.array_equal(a, b) for a, b in zip(again, (start, frm, to)))


def test_example_file_is_the_reference_example(tmp_path):
    path = str(tmp_path / 'v7e20.txt')
    graph.write_example_graph_to_text_file(path)
    assert np.array_equal(np.loadtxt(path, dtype=np.uint64).reshape(-1, 2), _golden('example')['pairs'])
    start, frm, to = graph.load_graph_from_text_file(path)
    assert graph.reference(start, frm, to) == 3


@pytest.mark.parametrize('name', ['example', 'random'])
def test_python_counter_and_oracle_match_the_reference(name):
    from oracle import runner
    g = _golden(name)
    start, frm, to = g['start'], g['from_vertex'], g['to_vertex']
    assert graph.reference(start, frm, to) == int(g['total'])
    per_edge = runner.evaluate([graph.triangles_op(start, frm, to)])
    assert per_edge.dtype == np.uint64 and np.array_equal(per_edge, g['per_edge'])


def test_counts_agree_with_the_adjacency_matrix():
    """trace(A^3) / 6 on a seeded random graph."""
    rs = np.random.RandomState(4)
    pairs = rs.randint(0, 60, size=(400, 2)).astype(np.uint64)
    start, frm, to = graph.adjacency_from_edges(pairs)
    a = np.zeros((len(start) - 1,) * 2, np.int64)
    a[frm.astype(np.int64), to.astype(np.int64)] = 1
    a = a + a.T
    assert graph.reference(start, frm, to) == int(np.trace(a @ a @ a)) // 6


@pytest.mark.gpu
@pytest.mark.parametrize('name', ['example', 'random'])
def test_gpu_counts_match_the_reference(name):
    import opveclib_b200 as ovl
    g = _golden(name)
    start, frm, to = g['start'], g['from_vertex'], g['to_vertex']
    per_edge = ovl.evaluate([graph.triangles_op(start, frm, to)], target_language='b200')
    total = graph.triangles(start, frm, to)
    if DRYRUN:
        pytest.skip('compiled; needs a device to run')
    assert np.array_equal(per_edge, g['per_edge'])
    assert total == int(g['total'])


@pytest.mark.gpu
def test_gpu_counts_on_a_larger_graph_match_the_oracle():
    import opveclib_b200 as ovl
    from oracle import runner
    rs = np.random.RandomState(9)
    pairs = rs.randint(0, 3000, size=(60000, 2)).astype(np.uint64)
    start, frm, to = graph.adjacency_from_edges(pairs)
    op = [graph.triangles_op(start, frm, to)]
    got = ovl.evaluate(op, target_language='b200')
    if DRYRUN:
        pytest.skip('compiled; needs a device to run')
    assert np.array_equal(got, runner.evaluate(op))
