"""Triangle counting in an undirected graph as an operator with data-dependent indexing and a bounded merge loop
(same interface and results as ``triangles_op`` / ``triangles`` / ``load_graph_from_text_file`` of
opveclib/examples/test_graph.py:16-101, 240-368).

The graph arrives as a compressed adjacency structure over ORIENTED edges (every undirected edge once, from its
higher-numbered to its lower-numbered end): ``startEdge[v] .. startEdge[v + 1]`` is the range of vertex v's edges in
``fromVertex`` / ``toVertex``, and the neighbours in each range are sorted.  One worker per edge (u, v) walks the
two sorted neighbour lists of u and v in step and counts the vertices that appear in both and are smaller than v;
with the orientation above every triangle is found at exactly one edge.  The walk is a ``while`` loop in spirit;
the operator language has counted loops only, so it runs for the combined length of the two lists and does
nothing once either list is exhausted.
"""
import numpy as np

from .. import expr as ovl
from ..opgraph import operator


@operator()
def triangles_op(startEdge, fromVertex, toVertex):
    """Per-edge triangle counts (uint64, one per entry of ``toVertex``)."""
    edge = ovl.position_in(toVertex.shape)[0]
    counts = ovl.output(toVertex.shape, ovl.uint64)
    # (a cursor that has run off its list is never used for a comparison, but it is used for a read: keep the read
    # inside the array)
    last_edge = toVertex.shape[0] - 1

    def neighbour(cursor):
        return toVertex[ovl.minimum(cursor, last_edge)]

    u = ovl.variable(fromVertex[edge], fromVertex.dtype)
    v = ovl.variable(toVertex[edge], toVertex.dtype)
    cur_u = ovl.variable(startEdge[u], startEdge.dtype)
    end_u = ovl.variable(startEdge[u + 1], startEdge.dtype)
    cur_v = ovl.variable(startEdge[v], startEdge.dtype)
    end_v = ovl.variable(startEdge[v + 1], startEdge.dtype)
    near_u = ovl.variable(neighbour(cur_u), toVertex.dtype)
    near_v = ovl.variable(neighbour(cur_v), toVertex.dtype)
    found = ovl.variable(0, ovl.uint64)

    longest_walk = (end_u - cur_u) + (end_v - cur_v)
    for _ in ovl.arange(longest_walk):
        in_lists = ovl.logical_and(cur_u < end_u, cur_v < end_v)
        with ovl.if_(ovl.logical_and(in_lists, near_u < v)):
            with ovl.if_(near_u < near_v):
                cur_u <<= cur_u + 1
                near_u <<= neighbour(cur_u)
            with ovl.elif_(near_u > near_v):
                cur_v <<= cur_v + 1
                near_v <<= neighbour(cur_v)
            with ovl.else_():
                found <<= found + 1
                cur_u <<= cur_u + 1
                cur_v <<= cur_v + 1
                near_u <<= neighbour(cur_u)
                near_v <<= neighbour(cur_v)
    counts[edge] = found
    return counts


def triangles(startEdge, fromVertex, toVertex, target_language='b200'):
    """Number of triangles of the graph: the operator's per-edge counts, summed on the host."""
    from ..runtime import evaluate
    per_edge = evaluate(triangles_op(startEdge, fromVertex, toVertex), target_language=target_language)
    if hasattr(per_edge, 'cpu'):
        per_edge = per_edge.cpu().numpy()
    return int(np.sum(per_edge, dtype=np.uint64))


def reference(startEdge, fromVertex, toVertex):
    """The same count in plain Python (sorted-list intersection per edge)."""
    if len(fromVertex) != len(toVertex):
        raise ValueError('fromVertex and toVertex must have one entry per edge each')
    total = 0
    for u, v in zip(fromVertex, toVertex):
        mine = toVertex[int(startEdge[int(u)]):int(startEdge[int(u) + 1])]
        theirs = toVertex[int(startEdge[int(v)]):int(startEdge[int(v) + 1])]
        i = j = 0
        while i < len(mine) and j < len(theirs) and mine[i] < v:
            if mine[i] < theirs[j]:
                i += 1
            elif mine[i] > theirs[j]:
                j += 1
            else:
                total += 1
                i += 1
                j += 1
    return total


def adjacency_from_edges(pairs):
    """(startEdge, fromVertex, toVertex), all uint64, from an array of vertex-id pairs.

    Ids are renumbered 0, 1, 2 ... in order of first appearance (reading the pairs row by row, first column first);
    self-loops and repeated edges (in either direction) are dropped; every remaining edge is kept once, from its
    higher to its lower number; edges are grouped by their first vertex with the neighbours of a group ascending."""
    pairs = np.asarray(pairs, dtype=np.uint64).reshape(-1, 2)
    flat = pairs.reshape(-1)
    ids, first_seen, inverse = np.unique(flat, return_index=True, return_inverse=True)
    rank_of_id = np.empty(len(ids), dtype=np.int64)
    rank_of_id[np.argsort(first_seen, kind='stable')] = np.arange(len(ids))
    renumbered = rank_of_id[inverse].reshape(-1, 2)
    # (the table of starts is sized by the largest id as given, like the reference's: ids that are not 0 .. V-1
    # leave vertices without edges at its end)
    vertices = int(flat.max()) + 1 if len(flat) else 0
    hi = renumbered.max(axis=1) if len(renumbered) else np.zeros(0, np.int64)
    lo = renumbered.min(axis=1) if len(renumbered) else np.zeros(0, np.int64)
    keep = hi != lo
    oriented = np.unique(np.stack([hi[keep], lo[keep]], axis=1), axis=0)      # sorted by (from, to), duplicates gone
    from_vertex = oriented[:, 0].astype(np.uint64)
    to_vertex = oriented[:, 1].astype(np.uint64)
    start = np.zeros(vertices + 1, dtype=np.uint64)
    start[1:] = np.cumsum(np.bincount(oriented[:, 0], minlength=vertices)).astype(np.uint64)
    return start, from_vertex, to_vertex


def load_graph_from_text_file(fileName):
    """Read an edge list (one ``from<TAB>to`` pair of integers per line, ``#`` starts a comment line) and return
    :func:`adjacency_from_edges` of it."""
    pairs = []
    with open(fileName, 'r') as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith('#'):
                continue
            tokens = line.split('\t')
            if len(tokens) != 2:
                raise ValueError('expected two tab-separated vertex ids, found: ' + line)
            pairs.append((int(tokens[0]), int(tokens[1])))
    return adjacency_from_edges(np.array(pairs, dtype=np.uint64).reshape(-1, 2))


def example_edges():
    """A graph of 7 vertices and 20 directed edges (10 undirected ones, each listed both ways) with 3 triangles:
    the ring 0-1-...-6-0 plus the chords 1-3, 3-5 and 1-6."""
    one_way = [(i, i + 1) for i in range(6)] + [(0, 6), (1, 3), (3, 5), (1, 6)]
    return one_way + [(b, a) for a, b in one_way]


def write_example_graph_to_text_file(fileName):
    """Write :func:`example_edges` as a tab-separated edge list."""
    with open(fileName, 'w') as f:
        for a, b in example_edges():
            f.write('%d\t%d\n' % (a, b))
