"""Random operator graphs for the fuzz tests: element-wise arithmetic with exact results (no libm), comparisons,
branches, broadcast-free binary operators, cyclic and affine index shifts, axis swaps on the reading and on the writing
side, strided gathers, clamped stencils, integer scans and reduction loops, stacking and unstacking along a new
axis.  Every graph is a pure function of its seed."""
import numpy as np


def _ops(ovl):
    @ovl.operator()
    def binary(a, b, fn=None):
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        x, y = a[pos], b[pos]
        if fn == 'add':
            out[pos] = x + y
        elif fn == 'sub':
            out[pos] = x - y
        elif fn == 'mul':
            out[pos] = x * y
        elif fn == 'min':
            out[pos] = ovl.minimum(x, y)
        elif fn == 'max':
            out[pos] = ovl.maximum(x, y)
        else:
            raise ValueError(fn)
        return out

    @ovl.operator()
    def affine(a, scale=None, shift=None):
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        out[pos] = a[pos] * scale + shift
        return out

    @ovl.operator()
    def select(a, b, c):
        # three-way branch with a store in every arm
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        with ovl.if_(a[pos] < b[pos]):
            out[pos] = c[pos]
        with ovl.elif_(a[pos] == b[pos]):
            out[pos] = a[pos] + c[pos]
        with ovl.else_():
            out[pos] = b[pos] - c[pos]
        return out

    @ovl.operator()
    def magnitude(a):
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        out[pos] = ovl.absolute(a[pos]) - a[pos] * a[pos]
        return out

    @ovl.operator()
    def rotate_last(a, k=None):
        # cyclic shift along the last axis: a permuting write
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        index = [pos[d] for d in range(a.rank)]
        index[-1] = (pos[a.rank - 1] + k) % a.shape[-1]
        out[index] = a[pos]
        return out

    @ovl.operator()
    def mirror_first(a):
        # reads the row mirrored along the first axis: an affine read with a negative coefficient
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        index = [pos[d] for d in range(a.rank)]
        index[0] = (a.shape[0] - 1) - pos[0]
        out[pos] = a[index]
        return out

    @ovl.operator()
    def stack_pair(a, b):
        out = ovl.output([2] + list(a.shape), a.dtype)
        pos = ovl.position_in(a.shape)
        out[[0] + [pos[d] for d in range(a.rank)]] = a[pos]
        out[[1] + [pos[d] for d in range(a.rank)]] = b[pos]
        return out

    @ovl.operator()
    def unstack_pair(s):
        shape = list(s.shape[1:])
        first, second = ovl.output(shape, s.dtype), ovl.output(shape, s.dtype)
        pos = ovl.position_in(shape)
        first[pos] = s[[0] + [pos[d] for d in range(len(shape))]]
        second[pos] = s[[1] + [pos[d] for d in range(len(shape))]]
        return first, second

    @ovl.operator()
    def row_total(a):
        # every worker sums its whole last-axis line: a loop with a loop-carried variable
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        total = ovl.variable(0, a.dtype)
        index = [pos[d] for d in range(a.rank)]
        for j in ovl.arange(a.shape[-1]):
            index[-1] = j
            total <<= total + a[index]
        out[pos] = total - a[pos]
        return out

    @ovl.operator()
    def gather_stride(a, k=None):
        # a strided gather with wrap-around along the last axis
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        index = [pos[d] for d in range(a.rank)]
        index[-1] = (pos[a.rank - 1] * k) % a.shape[-1]
        out[pos] = a[index]
        return out

    @ovl.operator()
    def neighbours(a):
        # a three-point stencil along the last axis with clamped ends
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        last = a.rank - 1
        left = [pos[d] for d in range(a.rank)]
        right = [pos[d] for d in range(a.rank)]
        left[last] = ovl.maximum(pos[last], 1) - 1
        right[last] = ovl.minimum(pos[last] + 1, a.shape[-1] - 1)
        out[pos] = a[left] - a[pos] + a[right]
        return out

    @ovl.operator()
    def swap_last_two(a):
        # reads its operand with the last two axes exchanged (square trailing axes keep the shape)
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        index = [pos[d] for d in range(a.rank)]
        index[-1], index[-2] = pos[a.rank - 2], pos[a.rank - 1]
        out[pos] = a[index]
        return out

    @ovl.operator()
    def scatter_last_two(a):
        # writes its result with the last two axes exchanged
        out = ovl.output_like(a)
        pos = ovl.position_in(a.shape)
        index = [pos[d] for d in range(a.rank)]
        index[-1], index[-2] = pos[a.rank - 2], pos[a.rank - 1]
        out[index] = a[pos] + a[pos]
        return out

    return dict(swap_last_two=swap_last_two, scatter_last_two=scatter_last_two, gather_stride=gather_stride, neighbours=neighbours, row_total=row_total, binary=binary, affine=affine, select=select, magnitude=magnitude, rotate_last=rotate_last,
                mirror_first=mirror_first, stack_pair=stack_pair, unstack_pair=unstack_pair)


_cache = {}


def build(ns, seed):
    """(outputs, leaf arrays) of the random graph with this seed."""
    ovl = ns.ovl
    if id(ovl) not in _cache:
        _cache[id(ovl)] = _ops(ovl)
    ops = _cache[id(ovl)]
    rs = np.random.RandomState(seed)
    rank = rs.randint(1, 4)
    shape = [int(rs.choice([1, 2, 3, 4, 5, 7, 8, 12, 16, 31, 33, 64, 100])) for _ in range(rank)]
    square = rank >= 2 and rs.rand() < 0.5
    if square:
        shape[-2] = shape[-1]
    dtype = rs.choice(['float32', 'float32', 'int32', 'float64', 'int16'])
    n_leaves = rs.randint(1, 4)
    if dtype.startswith('float'):
        leaves = [rs.uniform(-3, 3, shape).astype(dtype) for _ in range(n_leaves)]
    else:
        leaves = [rs.randint(-9, 10, shape).astype(dtype) for _ in range(n_leaves)]
    values = list(leaves)
    exact_sums = not dtype.startswith('float')      # integer sums do not depend on the order of evaluation
    kinds = ['binary', 'binary', 'binary', 'affine', 'select', 'magnitude', 'rotate', 'mirror', 'stack', 'gather',
             'neighbours']
    if square:
        kinds += ['swap', 'swap', 'scatter']
    if exact_sums:
        # no products of products (signed overflow), but scans and reduction loops
        kinds = [k for k in kinds if k != 'magnitude'] + ['cumsum', 'row_total']
    for _ in range(rs.randint(3, 12)):
        kind = rs.choice(kinds)
        pick = lambda: values[rs.randint(len(values))]     # noqa: E731
        if kind == 'binary':
            fns = ['add', 'sub', 'min', 'max'] + ([] if exact_sums else ['mul'])
            new = ops['binary'](pick(), pick(), fn=str(rs.choice(fns)))
        elif kind == 'affine':
            if dtype.startswith('float'):
                new = ops['affine'](pick(), scale=float(rs.choice([0.5, 2.0, -1.0, 0.25])), shift=float(rs.randint(-2, 3)))
            else:
                new = ops['affine'](pick(), scale=int(rs.randint(-2, 3)), shift=int(rs.randint(-2, 3)))
        elif kind == 'select':
            new = ops['select'](pick(), pick(), pick())
        elif kind == 'magnitude':
            new = ops['magnitude'](pick())
        elif kind == 'rotate':
            new = ops['rotate_last'](pick(), k=int(rs.randint(1, 5)))
        elif kind == 'cumsum':
            new = ns.cumsum(pick(), axis=int(rs.randint(rank)))
        elif kind == 'row_total':
            new = ops['row_total'](pick())
        elif kind == 'swap':
            new = ops['swap_last_two'](pick())
        elif kind == 'scatter':
            new = ops['scatter_last_two'](pick())
        elif kind == 'gather':
            new = ops['gather_stride'](pick(), k=int(rs.randint(2, 4)))
        elif kind == 'neighbours':
            new = ops['neighbours'](pick())
        elif kind == 'mirror':
            new = ops['mirror_first'](pick())
        else:
            pair = ops['unstack_pair'](ops['stack_pair'](pick(), pick()))
            values.append(pair[0])
            new = pair[1]
        values.append(new)
    produced = values[n_leaves:]
    count = min(len(produced), int(rs.randint(1, 4)))
    chosen = [produced[-1]] + [produced[i] for i in rs.choice(len(produced) - 1, size=count - 1, replace=False)] \
        if len(produced) > 1 else [produced[-1]]
    return chosen, leaves
