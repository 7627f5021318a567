"""Index analysis: which integer expressions of a kernel are affine functions of the worker position.

The operator language lets a worker read and write any element (opveclib/expression.py:859-973 builds the
linear offset from arbitrary scalar expressions).  Code generation and operator fusion need to know when an
offset is a *provably wrap-free* affine function ``const + sum(coef_d * position[d]) + sum(coef_v * loopvar_v)``:
then accesses of neighbouring workers are contiguous (vectorisable), two index expressions can be compared
exactly, and in-bounds-ness is decidable at compile time.  Integer arithmetic of the language wraps (uint32
position math); a form is only produced when interval arithmetic proves that no intermediate value leaves its
type's range, so the form equals the machine result for every worker.  ``(affine) % N`` with a constant N is
kept as a separate modular form (cyclic shifts).
"""
from . import expr as E
from .kernel import iter_nodes

_INT_RANGE = {
    'int8': (-2 ** 7, 2 ** 7 - 1), 'int16': (-2 ** 15, 2 ** 15 - 1), 'int32': (-2 ** 31, 2 ** 31 - 1),
    'int64': (-2 ** 63, 2 ** 63 - 1), 'uint8': (0, 2 ** 8 - 1), 'uint16': (0, 2 ** 16 - 1),
    'uint32': (0, 2 ** 32 - 1), 'uint64': (0, 2 ** 64 - 1),
}


class Affine(object):
    """const + sum(coef * symbol); symbols are ('p', dim) for position entries and ('l', n) for the n-th loop
    variable of the kernel.  ``mod`` (optional int) means the whole value is taken modulo ``mod``."""
    __slots__ = ('coefs', 'const', 'mod')

    def __init__(self, coefs=None, const=0, mod=None):
        self.coefs = {k: v for k, v in (coefs or {}).items() if v != 0}
        self.const = const
        self.mod = mod

    def is_const(self):
        return not self.coefs and self.mod is None

    def key(self):
        return (tuple(sorted(self.coefs.items())), self.const, self.mod)

    def __eq__(self, other):
        return isinstance(other, Affine) and self.key() == other.key()

    def __ne__(self, other):
        return not self == other

    def __hash__(self):
        return hash(self.key())

    def __repr__(self):
        return 'Affine(%r, %r, mod=%r)' % (self.coefs, self.const, self.mod)

    def coef(self, sym):
        return self.coefs.get(sym, 0)

    def bounds(self, ranges):
        """(min, max) over the symbol ranges (inclusive)."""
        if self.mod is not None:
            return 0, self.mod - 1
        lo = hi = self.const
        for sym, c in self.coefs.items():
            a, b = ranges[sym]
            lo += min(c * a, c * b)
            hi += max(c * a, c * b)
        return lo, hi

    def evaluate(self, values):
        v = self.const + sum(c * values[s] for s, c in self.coefs.items())
        return v % self.mod if self.mod is not None else v


class Access(object):
    """One tensor read or write of a kernel."""
    __slots__ = ('node', 'tensor', 'is_write', 'form', 'loop_depth', 'cond_depth')

    def __init__(self, node, tensor, is_write, form, loop_depth, cond_depth):
        self.node = node
        self.tensor = tensor
        self.is_write = is_write
        self.form = form
        self.loop_depth = loop_depth
        self.cond_depth = cond_depth


class KernelInfo(object):
    """Result of :func:`analyze`: ``forms`` maps id(node) -> Affine for every integer scalar with a proven
    form; ``accesses`` lists reads/writes of inputs, outputs and local tensors in program order; ``ranges`` maps
    symbols to inclusive value ranges (``steps``: the step of a loop symbol); ``loop_vars`` maps id(loop variable
    node) -> symbol."""

    def __init__(self):
        self.forms = {}
        self.accesses = []
        self.ranges = {}
        self.steps = {}
        self.loop_vars = {}
        self.assigned_vars = set()
        self.position_scalar_uses = 0

    def form_of(self, node):
        return self.forms.get(id(node))


def _fits(form, dtype, ranges):
    lo, hi = form.bounds(ranges)
    tlo, thi = _INT_RANGE[dtype.name]
    return tlo <= lo and hi <= thi


def analyze(kernel):
    info = KernelInfo()
    shape = kernel.workgroup_shape
    for d, n in enumerate(shape):
        info.ranges[('p', d)] = (0, n - 1)

    # variables assigned anywhere are mutable unless they are the induction variable of exactly one loop
    assign_count = {}
    for node in iter_nodes(kernel.body):
        if node.kind == 'assign_var':
            assign_count[id(node.args[0])] = assign_count.get(id(node.args[0]), 0) + 1
    info.assigned_vars = set(assign_count)

    def visit(block, loop_depth, cond_depth):
        for node in block.nodes:
            k = node.kind
            if k == 'const':
                if isinstance(node.attr['value'], int):
                    info.forms[id(node)] = Affine(const=node.attr['value'])
            elif k == 'cast':
                src = info.forms.get(id(node.args[0]))
                if src is not None and not node.dtype.is_float and _fits(src, node.dtype, info.ranges):
                    info.forms[id(node)] = src
            elif k == 'variable':
                # a variable nobody assigns to is a named constant (e.g. a loop bound taken from a shape)
                src = info.forms.get(id(node.args[0]))
                if (src is not None and id(node) not in assign_count and not node.dtype.is_float
                        and _fits(src, node.dtype, info.ranges)):
                    info.forms[id(node)] = src
            elif k == 'read':
                tensor, index = node.args
                iform = info.forms.get(id(index))
                if tensor.kind == 'position':
                    if iform is not None and iform.is_const():
                        info.forms[id(node)] = Affine({('p', iform.const): 1})
                else:
                    info.accesses.append(Access(node, tensor, False, iform, loop_depth, cond_depth))
            elif k == 'assign_tensor':
                tensor, index = node.args[0], node.args[1]
                info.accesses.append(Access(node, tensor, True, info.forms.get(id(index)), loop_depth,
                                            cond_depth))
            elif k == 'binary' and not node.dtype.is_float:
                a = info.forms.get(id(node.args[0]))
                b = info.forms.get(id(node.args[1]))
                fn = node.attr['fn']
                res = None
                if a is not None and b is not None and a.mod is None and b.mod is None:
                    if fn == 'add':
                        coefs = dict(a.coefs)
                        for s, c in b.coefs.items():
                            coefs[s] = coefs.get(s, 0) + c
                        res = Affine(coefs, a.const + b.const)
                    elif fn == 'sub':
                        coefs = dict(a.coefs)
                        for s, c in b.coefs.items():
                            coefs[s] = coefs.get(s, 0) - c
                        res = Affine(coefs, a.const - b.const)
                    elif fn == 'mul' and (a.is_const() or b.is_const()):
                        c, f = (a.const, b) if a.is_const() else (b.const, a)
                        res = Affine({s: v * c for s, v in f.coefs.items()}, f.const * c)
                    elif fn == 'mod' and b.is_const() and b.const > 0:
                        lo, hi = a.bounds(info.ranges)
                        if 0 <= lo and hi < b.const:
                            res = a
                        elif lo >= 0:
                            res = Affine(a.coefs, a.const, mod=b.const)
                elif a is not None and b is not None and fn == 'mul':
                    # a modular form survives multiplication by one (row-major stride of a rank-1 tensor)
                    if a.mod is not None and b.is_const() and b.const == 1:
                        res = a
                    elif b.mod is not None and a.is_const() and a.const == 1:
                        res = b
                elif a is not None and b is not None and fn == 'add':
                    if a.mod is not None and b.is_const() and b.const == 0:
                        res = a
                    elif b.mod is not None and a.is_const() and a.const == 0:
                        res = b
                if res is not None and _fits(res, node.dtype, info.ranges):
                    info.forms[id(node)] = res
            elif k == 'for':
                var, start, stop, step = node.args
                fs, fe, fst = (info.forms.get(id(x)) for x in (start, stop, step))
                sym = None
                if (fs is not None and fe is not None and fst is not None and fs.is_const() and fe.is_const()
                        and fst.is_const() and fst.const != 0 and assign_count.get(id(var), 0) == 0
                        and id(var) not in info.loop_vars and not var.dtype.is_float):
                    s, e, st = fs.const, fe.const, fst.const
                    trips = max(0, -(-(e - s) // st)) if st > 0 else max(0, -(-(s - e) // (-st)))
                    if trips > 0:
                        last = s + (trips - 1) * st
                        sym = ('l', len(info.loop_vars))
                        info.loop_vars[id(var)] = sym
                        info.ranges[sym] = (min(s, last), max(s, last))
                        info.steps[sym] = st
                        info.forms[id(var)] = Affine({sym: 1})
                visit(node.body, loop_depth + 1, cond_depth)
                if sym is not None:
                    # after the loop the variable holds the exit value; it is no longer the induction symbol
                    del info.forms[id(var)]
            elif k == 'if':
                for blk in node.blocks:
                    visit(blk, loop_depth, cond_depth + 1)

    visit(kernel.body, 0, 0)
    return info
