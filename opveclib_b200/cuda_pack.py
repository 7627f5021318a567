"""Packed body emission for the ``math='tolerance'`` lowering: two workers per expression.

A vectorised fp32 kernel gives each thread four consecutive workers.  When the body is pure fp32 element-wise
arithmetic - every tensor access hoisted into the group's vector loads and stores, no loops, no worker-local
tensors, no integer values that feed results - the four workers can be evaluated as two pairs whose additions,
multiplications and fused multiply-adds are single ``*.f32x2`` instructions (``ovl::tol::f2`` in
csrc/templates/ovl_fastmath.cuh).  Conditionals lose their branches: every branch of an ``if_/elif_/else_`` chain is
evaluated for both workers of a pair.  A chain whose branches do nothing but assign one and the same variable (or
output) becomes one nested select, ``c0 ? v0 : (c1 ? v1 : ...)``; in any other chain the assignments keep the old
value where the branch's condition does not hold for a worker (masks).  Results are unchanged either way because
branches may only assign variables and hoisted outputs.

``plan_pairs`` decides whether a kernel qualifies; ``PairEmitter`` writes the body.  Statement order, operand
types and rounding points are those of the scalar body (opveclib/expression.py:559-566 and the per-node
``gen_c``): each +, -, * is one rounded operation, nothing is contracted.
"""
from .kernel import iter_nodes

_T = 'ovl::tol::'
_ARITH = {'add': 'add2', 'sub': 'sub2', 'mul': 'mul2', 'div': 'fdiv', 'eq': 'eq2', 'ne': 'ne2', 'lt': 'lt2',
          'le': 'le2', 'gt': 'gt2', 'ge': 'ge2', 'and': 'and2', 'or': 'or2', 'min': 'min2', 'max': 'max2'}
_BINARY_LIBM = {'pow': 'powf', 'atan2': 'atan2f', 'mod': 'fmodf'}
_UNARY = {'negate': 'neg2', 'not': 'not2', 'abs': 'abs2', 'isinf': 'isinf2', 'isnan': 'isnan2',
          'isfinite': 'isfinite2', 'exp': 'fexp', 'log': 'flog', 'tanh': 'ftanh', 'log10': 'flog10',
          'sqrt': 'fsqrt'}
_UNARY_LIBM = {'acos': 'acosf', 'asin': 'asinf', 'atan': 'atanf', 'cos': 'cosf', 'cosh': 'coshf', 'sin': 'sinf',
               'sinh': 'sinhf', 'tan': 'tanf', 'ceil': 'ceilf', 'floor': 'floorf'}


def _is_f32(node):
    return getattr(node, 'is_scalar', False) and node.dtype.name == 'float32'


def plan_pairs(kernel, plan):
    """The set of node ids the paired body must evaluate, or None when the kernel does not qualify.

    ``plan`` is the kernel's vectorisation plan: reads and writes it hoists are the only tensor accesses a paired
    body may contain."""
    if plan.lanes < 2 or plan.lanes % 2:
        return None
    hoisted_reads = set(id(n) for slot in plan.read_slots for n in slot[3])
    hoisted_writes = set(id(n) for slot in plan.write_slots for n in slot[2])
    needed = {}
    stack = []

    def want(node):
        if id(node) not in needed:
            needed[id(node)] = node
            stack.append(node)

    for node in iter_nodes(kernel.body):
        k = node.kind
        if k in ('for', 'local'):       # (constant tensors only ever initialise worker-local tensors)
            return None
        if k == 'assign_tensor':
            if id(node) not in hoisted_writes:
                return None
            want(node.args[2])
        elif k == 'assign_var':
            want(node.args[0])
            want(node.args[1])
        elif k == 'if':
            for cond in node.conds:
                if cond is not None:
                    want(cond)
    while stack:
        node = stack.pop()
        k = node.kind
        if not _is_f32(node):
            return None
        if k == 'read':
            if id(node) not in hoisted_reads:
                return None
            continue
        if k in ('variable', 'cast'):
            src = node.args[0]
            if src.kind == 'const':
                continue
            if k == 'variable' or not _is_f32(src):
                return None
            want(src)
        elif k in ('unary', 'binary'):
            for a in node.args:
                want(a)
        elif k != 'limit':
            return None
    return set(needed)


class PairEmitter(object):
    """Emits a kernel body over pairs of workers.  ``read_text`` maps id(read node) to the C text of its pair of
    values; ``write_name`` maps id(assign node) to the name of the ``f2`` that collects the pair to be stored."""

    def __init__(self, kernel, indent, needed, read_text, write_name, literal, limits):
        self.kernel = kernel
        self.needed = needed
        self.read_text = read_text
        self.write_name = write_name
        self.literal = literal
        self.limits = limits
        self.names = {}
        self.lines = []
        self.depth = indent
        self.counter = 0
        self.mask = None

    def put(self, text):
        self.lines.append('    ' * self.depth + text)

    def fresh(self, node=None, prefix='e'):
        n = prefix + str(self.counter)
        self.counter += 1
        if node is not None:
            self.names[id(node)] = n
        return n

    def name(self, node):
        return self.names[id(node)]

    def _splat_const(self, node):
        return _T + 'splat((float)(' + self.literal(node.attr['value']) + '))'

    def block(self, block):
        for node in block.nodes:
            self.node(node)

    def _assign(self, target, value):
        if self.mask is None:
            self.put(target + ' = ' + value + ';')
        else:
            self.put(target + ' = ' + _T + 'pick(' + self.mask + ', ' + value + ', ' + target + ');')

    def node(self, node):
        k = node.kind
        if k == 'assign_tensor':
            self._assign(self.write_name[id(node)], self.name(node.args[2]))
            return
        if k == 'assign_var':
            self._assign(self.name(node.args[0]), self.name(node.args[1]))
            return
        if k == 'if':
            self._if(node)
            return
        if id(node) not in self.needed:
            return
        decl = _T + 'f2 '
        if k == 'read':
            self.put(decl + self.fresh(node) + ' = ' + self.read_text[id(node)] + ';')
        elif k == 'variable':
            self.put(decl + self.fresh(node) + ' = ' + self._splat_const(node.args[0]) + ';')
        elif k == 'cast':
            src = node.args[0]
            rhs = self._splat_const(src) if src.kind == 'const' else self.name(src)
            self.put('const ' + decl + self.fresh(node) + ' = ' + rhs + ';')
        elif k == 'limit':
            self.put('const ' + decl + self.fresh(node) + ' = ' + _T + 'splat(' +
                     self.limits[(node.attr['which'], 'float32')] + ');')
        elif k == 'unary':
            fn = node.attr['fn']
            x = self.name(node.args[0])
            if fn in _UNARY:
                rhs = _T + _UNARY[fn] + '(' + x + ')'
            else:
                f = _UNARY_LIBM[fn]
                rhs = _T + 'make2(' + f + '(' + x + '.x), ' + f + '(' + x + '.y))'
            self.put('const ' + decl + self.fresh(node) + ' = ' + rhs + ';')
        elif k == 'binary':
            fn = node.attr['fn']
            whole = self._positive_infinity_test(node)
            if whole is not None:
                self.put('const ' + decl + self.fresh(node) + ' = ' + _T + 'isposinf2(' + self.name(whole) + ');')
                return
            x, y = self.name(node.args[0]), self.name(node.args[1])
            if fn in _ARITH:
                rhs = _T + _ARITH[fn] + '(' + x + ', ' + y + ')'
            else:
                f = _BINARY_LIBM[fn]
                rhs = _T + 'make2(' + f + '(' + x + '.x, ' + y + '.x), ' + f + '(' + x + '.y, ' + y + '.y))'
            self.put('const ' + decl + self.fresh(node) + ' = ' + rhs + ';')
        else:
            raise NotImplementedError(k)

    @staticmethod
    def _positive_infinity_test(node):
        """``v`` when the node is ``logical_and(isinf(v), v > 0)`` (either order) - the guard the example operators
        put in front of their formulas - which is the single comparison ``v == +inf``."""
        if node.attr['fn'] != 'and':
            return None

        def source(n):          # through same-type copies of a variable or value
            while n.kind == 'cast' and n.args[0].kind != 'const' and n.args[0].dtype == n.dtype:
                n = n.args[0]
            return n
        for a, b in (node.args, node.args[::-1]):
            if a.kind == 'unary' and a.attr['fn'] == 'isinf' and b.kind == 'binary' and b.attr['fn'] == 'gt':
                zero = b.args[1]
                if zero.kind == 'cast' and zero.args[0].kind == 'const' and zero.args[0].attr['value'] == 0 and \
                        source(a.args[0]) is source(b.args[0]):
                    return a.args[0]
        return None

    _PURE = ('const', 'read', 'cast', 'unary', 'binary', 'limit')

    def _single_target(self, node):
        """The C name of the one variable (or output pair) that every branch of the chain assigns exactly once, with
        nothing else in the branches but value computations; None for any other chain."""
        target = None
        for blk in node.blocks:
            effects = [n for n in blk.nodes if n.kind not in self._PURE]
            if len(effects) != 1:
                return None
            e = effects[0]
            if e.kind == 'assign_var':
                name = self.name(e.args[0])
            elif e.kind == 'assign_tensor':
                name = self.write_name[id(e)]
            else:
                return None
            if target is not None and name != target:
                return None
            target = name
        return target

    def _if(self, node):
        target = self._single_target(node)
        if target is not None:
            # value = c0 ? v0 : (c1 ? v1 : ... : value): one select per branch and no mask arithmetic
            values = []
            for blk in node.blocks:
                for n in blk.nodes:
                    if n.kind in self._PURE:
                        self.node(n)
                    else:
                        values.append(self.name(n.args[2] if n.kind == 'assign_tensor' else n.args[1]))
            expr = target
            for cond, v in reversed(list(zip(node.conds, values))):
                expr = v if cond is None else _T + 'pick(' + _T + 'truth(' + self.name(cond) + '), ' + v + ', ' + expr + ')'
            self._assign(target, expr)
            return
        outer = self.mask
        rest = outer            # workers of the pair that no earlier branch of this chain has taken
        for cond, blk in zip(node.conds, node.blocks):
            if cond is not None:
                t = self.fresh(prefix='t')
                self.put('const ' + _T + 'b2 ' + t + ' = ' + _T + 'truth(' + self.name(cond) + ');')
                if rest is None:
                    taken = t
                else:
                    taken = self.fresh(prefix='m')
                    self.put('const ' + _T + 'b2 ' + taken + ' = ' + _T + 'both(' + rest + ', ' + t + ');')
                left = self.fresh(prefix='m')
                if rest is None:
                    self.put('const ' + _T + 'b2 ' + left + ' = ' + _T + 'andnot(' + _T + 'b2{true, true}, ' + t + ');')
                else:
                    self.put('const ' + _T + 'b2 ' + left + ' = ' + _T + 'andnot(' + rest + ', ' + t + ');')
                rest = left
            else:
                taken = rest
            self.mask = taken
            self.block(blk)
        self.mask = outer
