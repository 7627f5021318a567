"""CUDA code generation for sm_100a.

Every (fused) kernel is lowered to a ``.cu`` translation unit that instantiates hand-written templates from
``csrc/templates`` with the kernel's body.  The body is emitted as straight-line C, one statement per
expression, in trace order and with each expression's own C type - the form the reference's generator emits
(opveclib/expression.py:559-566 and the per-node ``gen_c``), so that fp32 arithmetic rounds at the same places
as in the reference's C++ operator.  Code is compiled with ``--fmad=false`` and without fast-math; the
differences to the C++ build that remain are those of CUDA's libm (expf, logf, tanhf ... within 1-2 ulp).

Two entry points are generated per kernel:

``<name>_gen``  one worker per loop iteration of a grid-stride loop; scalar accesses exactly as written.  The
                correctness net for every access pattern (arbitrary scatter, loops, worker-local tensors).
``<name>_vec``  each thread owns ``LANES`` consecutive workers along the innermost workgroup axis.  Reads and
                writes whose offset is a wrap-free affine function of the position with unit stride along that
                axis are hoisted out of the body into 128-bit ``ld.global.nc`` / ``st.global`` of the whole
                group; offsets that do not depend on the innermost axis are loaded once per group; everything
                else stays a scalar access in place.  Chosen at launch when every hoisted tensor's base pointer
                is 16-byte aligned.

Scans recognised by :mod:`opveclib_b200.patterns` use the cooperative scan template instead.
"""
import math
import os

from . import expr as E
from .access import analyze, Affine
from .kernel import iter_nodes
from . import cuda_pack
from . import patterns

_UNARY_F32 = {'acos': 'acosf', 'asin': 'asinf', 'atan': 'atanf', 'cos': 'cosf', 'cosh': 'coshf', 'sin': 'sinf',
              'sinh': 'sinhf', 'tan': 'tanf', 'tanh': 'tanhf', 'exp': 'expf', 'log': 'logf', 'log10': 'log10f',
              'sqrt': 'sqrtf', 'ceil': 'ceilf', 'floor': 'floorf', 'abs': 'fabsf'}
_UNARY_F64 = {'acos': 'acos', 'asin': 'asin', 'atan': 'atan', 'cos': 'cos', 'cosh': 'cosh', 'sin': 'sin',
              'sinh': 'sinh', 'tan': 'tan', 'tanh': 'tanh', 'exp': 'exp', 'log': 'log', 'log10': 'log10',
              'sqrt': 'sqrt', 'ceil': 'ceil', 'floor': 'floor', 'abs': 'fabs'}
_ABS_INT = {'int8': 'ovl::abs_8', 'int16': 'ovl::abs_16', 'int32': 'abs', 'int64': 'llabs'}
_INFIX = {'add': '+', 'sub': '-', 'mul': '*', 'div': '/', 'mod': '%', 'eq': '==', 'ne': '!=', 'lt': '<',
          'le': '<=', 'gt': '>', 'ge': '>=', 'and': '&&', 'or': '||'}
# math='tolerance': fp32 division and these fp32 functions go to csrc/templates/ovl_fastmath.cuh
_TOLERANCE_F32 = {'exp': 'ovl::tol::fexp', 'log': 'ovl::tol::flog', 'tanh': 'ovl::tol::ftanh',
                  'log10': 'ovl::tol::flog10', 'sqrt': 'ovl::tol::fsqrt'}
MATH_MODES = ('exact', 'tolerance')
_LIMITS = {('min_value', 'float32'): 'FLT_MIN', ('min_value', 'float64'): 'DBL_MIN',
           ('max_value', 'float32'): 'FLT_MAX', ('max_value', 'float64'): 'DBL_MAX',
           ('epsilon', 'float32'): 'FLT_EPSILON', ('epsilon', 'float64'): 'DBL_EPSILON'}

TEMPLATE_VERSION = 'tv45'
BLOCK_THREADS = 256
# must match kScanBlock / kScanVpt of csrc/templates/ovl_scan.cuh
SCAN_BLOCK = 512
SCAN_VPT = 4
SCAN_HEADER_BYTES = 16
# must match kRingThreads / kRingSlots / kRingCtlBytes / kRingMaxGrid of csrc/templates/ovl_scan.cuh
RING_THREADS = 864
RING_SLOTS = 6
RING_CTL_BYTES = 4096
RING_MAX_GRID = 256
# must match kColBlock / kColRows of csrc/templates/ovl_colscan.cuh
COL_BLOCK = 256
COL_ROWS = 64
COL_WALK_REGS = 32            # registers a lane spends on the rows it holds per tile of the one-launch column scan
COL_WALK_MIN_STRIPS = 148     # ... which needs at least a strip of columns per SM
WARP_SCAN_BLOCK = 256
WARP_SCAN_MIN_LINES = 2048     # from this many lines on, a warp scans a whole line by itself
WARP_SCAN_MIN_AXIS = 64        # ... if the line is at least this long
TILE_EDGE = 32                # smallest extent of the two tiled axes for which accesses are staged
TILE_WIDE = 64                # tile edge along an axis that is at least this long (32 otherwise)
TILE_SMEM_LIMIT = 40 * 1024   # bytes of shared memory the staged tiles of one kernel may take
# reduction loops: threads that share one worker's loop - a warp, or a whole block when there are too few workers
# to fill the device with warps and the loop is long enough to feed a block
REDUCE_BLOCK = 256
REDUCE_BLOCK_TRIPS = 2048
REDUCE_FEW_WORKERS = 2048
REDUCE_ACROSS_WIDE_BELOW = 1184      # blocks of 32 workers: fewer than eight per SM get 1024 threads each
REDUCE_SPLIT_MAX_WORKERS = 592       # block-per-worker loops of so few workers are cut into slices ...
REDUCE_SPLIT_MIN_TRIPS = 1 << 16     # ... when they are at least this long,
REDUCE_SPLIT_SLICE = 1 << 14         # into slices of at least this many trips
REDUCE_SPLIT_MAX = 2048              # (at most this many per worker)


def ctype(dtype):
    return dtype.as_cstr()


def literal(value):
    if isinstance(value, float):
        if math.isinf(value):
            return 'INFINITY' if value > 0 else '(-INFINITY)'
        if math.isnan(value):
            return 'NAN'
        return repr(value)
    v = int(value)
    if v > 2 ** 63 - 1:
        return str(v) + 'ull'
    if v == -2 ** 63:
        return '(-9223372036854775807ll - 1)'
    if abs(v) > 2 ** 31 - 1:
        return str(v) + 'll'
    return str(v)


class BodyEmitter(object):
    """Emits the statements of a kernel body.  ``read_subst`` / ``write_subst`` map id(node) of hoisted accesses
    to the C text that replaces the memory access (a register expression / an assignment template)."""

    def __init__(self, kernel, indent, read_subst=None, write_subst=None, position_text=None, math='exact'):
        self.kernel = kernel
        self.math = math
        self.names = {}
        self.lines = []
        self.depth = indent
        self.counter = 0
        self.read_subst = read_subst or {}
        self.write_subst = write_subst or {}
        self.position_text = position_text

    def name(self, node):
        return self.names[id(node)]

    def put(self, text):
        self.lines.append('    ' * self.depth + text)

    def fresh(self, node):
        n = 'e' + str(self.counter)
        self.counter += 1
        self.names[id(node)] = n
        return n

    def block(self, block):
        for node in block.nodes:
            self.node(node)

    def node(self, node):
        k = node.kind
        if k == 'input':
            self.names[id(node)] = 'in' + str(node.attr['io_index'])
        elif k == 'output':
            self.names[id(node)] = 'out' + str(node.attr['io_index'])
        elif k == 'const':
            self.names[id(node)] = literal(node.attr['value'])
        elif k == 'const_tensor':
            self.names[id(node)] = '{' + ', '.join(literal(v) for v in node.to_array().tolist()) + '}'
        elif k == 'position':
            self.names[id(node)] = 'position'
            if self.position_text is not None:
                self.put(self.position_text)
        elif k == 'variable' or k == 'cast':
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + ' = ' + self.name(node.args[0]) + ';')
        elif k == 'local':
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + '[' + str(node.size) + '] = ' + self.name(node.args[0]) + ';')
        elif k == 'assign_var':
            self.put(self.name(node.args[0]) + ' = ' + self.name(node.args[1]) + ';')
        elif k == 'assign_tensor':
            if id(node) in self.write_subst:
                self.put(self.write_subst[id(node)].replace('{index}', self.name(node.args[1])) % self.name(node.args[2]))
            else:
                self.put(self.name(node.args[0]) + '[' + self.name(node.args[1]) + '] = ' +
                         self.name(node.args[2]) + ';')
        elif k == 'read':
            n = self.fresh(node)
            if id(node) in self.read_subst:
                # ('{index}' in the text stands for the linear offset the read was traced with)
                self.put(ctype(node.dtype) + ' ' + n + ' = ' +
                         self.read_subst[id(node)].replace('{index}', self.name(node.args[1])) + ';')
            else:
                self.put(ctype(node.dtype) + ' ' + n + ' = ' + self.name(node.args[0]) + '[' +
                         self.name(node.args[1]) + '];')
        elif k == 'limit':
            self.names[id(node)] = _LIMITS[(node.attr['which'], node.dtype.name)]
        elif k == 'unary':
            fn, t = node.attr['fn'], node.dtype.name
            x = self.name(node.args[0])
            if fn == 'negate':
                rhs = '-(' + x + ')'
            elif fn == 'not':
                rhs = '!(' + x + ')'
            elif fn in ('isinf', 'isfinite', 'isnan'):
                # the host's std::isinf & co. return bool; CUDA's may return any non-zero int
                rhs = '(' + fn + '(' + x + ') ? 1 : 0)'
            elif fn == 'abs' and t in _ABS_INT:
                rhs = _ABS_INT[t] + '(' + x + ')'
            elif self.math == 'tolerance' and t == 'float32' and fn in _TOLERANCE_F32:
                rhs = _TOLERANCE_F32[fn] + '(' + x + ')'
            else:
                rhs = (_UNARY_F32 if t == 'float32' else _UNARY_F64)[fn] + '(' + x + ')'
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + ' = ' + rhs + ';')
        elif k == 'binary':
            fn, t = node.attr['fn'], node.dtype.name
            x, y = self.name(node.args[0]), self.name(node.args[1])
            if fn == 'min':
                rhs = '(((' + x + ')<(' + y + '))?(' + x + '):(' + y + '))'
            elif fn == 'max':
                rhs = '(((' + x + ')>(' + y + '))?(' + x + '):(' + y + '))'
            elif fn == 'pow':
                rhs = ('powf(' if t == 'float32' else 'pow(') + x + ',' + y + ')'
            elif fn == 'atan2':
                rhs = ('atan2f(' if t == 'float32' else 'atan2(') + x + ',' + y + ')'
            elif fn == 'mod' and t == 'float32':
                rhs = 'fmodf(' + x + ',' + y + ')'
            elif fn == 'mod' and t == 'float64':
                rhs = 'fmod(' + x + ',' + y + ')'
            elif fn == 'div' and t == 'float32' and self.math == 'tolerance':
                rhs = 'ovl::tol::fdiv(' + x + ', ' + y + ')'
            else:
                rhs = '(' + x + ' ' + _INFIX[fn] + ' ' + y + ')'
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + ' = ' + rhs + ';')
        elif k == 'for':
            i, a, b, s = [self.name(x) for x in node.args]
            self.put('for(' + i + ' = ' + a + '; ((' + i + ' < ' + b + ')&&(' + s + '>0)) || ((' + i + ' > ' + b +
                     ')&&(' + s + '<0)); ' + i + '+=' + s + '){')
            self.depth += 1
            self.block(node.body)
            self.depth -= 1
            self.put('}')
        elif k == 'if':
            for bi, (cond, blk) in enumerate(zip(node.conds, node.blocks)):
                if bi == 0:
                    self.put('if(' + self.name(cond) + '){')
                elif cond is not None:
                    self.put('}')
                    self.put('else if(' + self.name(cond) + '){')
                else:
                    self.put('}')
                    self.put('else{')
                self.depth += 1
                self.block(blk)
                self.depth -= 1
            self.put('}')
        else:
            raise NotImplementedError(k)


def _strides(shape):
    blocks = [1]
    for d in range(len(shape) - 1, 0, -1):
        blocks.append(blocks[-1] * shape[d])
    blocks.reverse()
    return blocks


def _position_values(shape, widx):
    """C expressions of the position entries of worker ``widx`` (opveclib/expression.py:1293-1306)."""
    vals, rem = [], widx
    for b in _strides(shape):
        vals.append('(uint32_t)((' + rem + ')/' + str(b) + 'u)')
        rem = '(' + rem + ') % ' + str(b) + 'u'
    return vals


def _params(kernel):
    params = []
    for n in kernel.inputs:
        params.append('const ' + ctype(n.dtype) + '* __restrict__ in' + str(n.attr['io_index']))
    for n in kernel.outputs:
        params.append(ctype(n.dtype) + '* __restrict__ out' + str(n.attr['io_index']))
    return params


def _is_injective(form, ranges):
    """Do distinct positions give distinct offsets?  (mixed-radix test on the coefficients)"""
    terms = sorted((abs(c), ranges[s][1] - ranges[s][0]) for s, c in form.coefs.items())
    span = 0
    for c, extent in terms:
        if extent == 0:
            continue
        if c <= span:
            return False
        span += c * extent
    return True


class VecPlan(object):
    """Which accesses of a kernel are hoisted into vector / uniform loads and vector stores."""

    def __init__(self):
        self.lanes = 0
        self.read_slots = []    # (tensor node, form, mode 'vec'|'uni', [read nodes])
        self.write_slots = []   # (tensor node, form, [assign nodes], conditional)

    @property
    def usable(self):
        return self.lanes > 1 and (any(s[2] == 'vec' for s in self.read_slots) or self.write_slots)


def plan_vectorisation(kernel, info=None):
    info = info or analyze(kernel)
    plan = VecPlan()
    shape = kernel.workgroup_shape
    last = len(shape) - 1
    psym = ('p', last)
    if shape[last] == 1:
        return plan
    io_nodes = [n for n in kernel.inputs + kernel.outputs]
    if not io_nodes:
        return plan

    def candidate(acc):
        f = acc.form
        if f is None or f.mod is not None or acc.loop_depth > 0:
            return None
        if any(s[0] == 'l' for s in f.coefs):
            return None
        if acc.tensor.kind not in ('input', 'output'):
            return None
        lo, hi = f.bounds(info.ranges)
        if lo < 0 or hi >= acc.tensor.size:
            return None
        c = f.coef(psym)
        if c == 1:
            return 'vec'
        if c == 0 and not acc.is_write:
            return 'uni'
        return None

    cands = [(acc, candidate(acc)) for acc in info.accesses]
    widest = max([acc.tensor.dtype.itemsize for acc, mode in cands if mode == 'vec'] or [0])
    if widest == 0:
        return plan
    lanes = max(1, 16 // widest)
    while lanes > 1 and shape[last] % lanes != 0:
        lanes //= 2
    if lanes <= 1:
        return plan

    def aligned(f):
        if f.const % lanes != 0:
            return False
        for s, c in f.coefs.items():
            if s != psym and c % lanes != 0 and info.ranges[s][1] > 0:
                return False
        return True

    reads, writes = {}, {}
    for acc, mode in cands:
        if mode is None:
            continue
        if mode == 'vec' and not aligned(acc.form):
            continue
        key = (id(acc.tensor), acc.form.key())
        if acc.is_write:
            writes.setdefault(key, [acc.tensor, acc.form, [], False])
            writes[key][2].append(acc.node)
            if acc.cond_depth > 0:
                writes[key][3] = True
        else:
            reads.setdefault(key, [acc.tensor, acc.form, mode, []])
            reads[key][3].append(acc.node)

    # a conditional store may only be widened to the whole group when no other worker and no other statement
    # can target the elements a skipped lane would have written
    slots_per_tensor = {}
    for acc in info.accesses:
        if acc.is_write and acc.tensor.kind == 'output':
            k = acc.form.key() if acc.form is not None else ('?', id(acc.node))
            slots_per_tensor.setdefault(id(acc.tensor), set()).add(k)
    for key, slot in list(writes.items()):
        if slot[3]:
            if len(slots_per_tensor[id(slot[0])]) != 1 or not _is_injective(slot[1], info.ranges):
                del writes[key]

    plan.lanes = lanes
    plan.read_slots = [tuple(v) for v in reads.values()]
    plan.write_slots = [tuple(v) for v in writes.values()]
    return plan


def _tile_edges(shape, axis, wide):
    """Tile extents along the staged axis and along the innermost axis."""
    if not wide:
        return TILE_EDGE, TILE_EDGE
    return (TILE_WIDE if shape[axis] >= TILE_WIDE else TILE_EDGE,
            TILE_WIDE if shape[-1] >= TILE_WIDE else TILE_EDGE)


ROWS_BLOCK = 128                     # workers (= rows) per block of a row-staged kernel
ROWS_MAX_ROW_BYTES = 1024
ROWS_MAX_SMEM = 200 * 1024


def plan_row_staging(kernel, info):
    """Input tensors that every worker reads only inside ITS OWN ROW - a run of ``rowlen`` consecutive elements that
    starts at rowlen * (linear worker index) - with at least one such read inside a loop (``acc += a[row, i]``,
    ``best = max(best, a[row, i])`` ...).  One thread per worker then walks through memory with a stride of a whole row
    and a warp's loads scatter over 32 rows; staging the rows of a block's workers in shared memory first (they are one
    contiguous piece of memory) makes the global reads coalesced and leaves the body, statement order and arithmetic
    as they are.  Returns a list of (tensor, rowlen, padded row length in elements, read nodes) or []."""
    shape = kernel.workgroup_shape
    strides = _strides(shape)
    W = 1
    for n in shape:
        W *= n
    by_tensor = {}
    for acc in info.accesses:
        if acc.tensor.kind == 'input' and not acc.is_write:
            by_tensor.setdefault(id(acc.tensor), (acc.tensor, []))[1].append(acc)
    staged, smem = [], 0
    for tensor, accs in by_tensor.values():
        size = tensor.size
        if W < 2 * ROWS_BLOCK or size % W:
            continue
        rowlen = size // W
        itemsize = tensor.dtype.itemsize
        if rowlen < 2 or rowlen * itemsize > ROWS_MAX_ROW_BYTES:
            continue
        ok, in_loop = True, False
        for acc in accs:
            f = acc.form
            if f is None or f.mod is not None:
                ok = False
                break
            rest = {}
            for sym, c in f.coefs.items():
                if sym[0] != 'p':
                    rest[sym] = c
            if any(f.coef(('p', d)) != rowlen * strides[d] for d, n in enumerate(shape) if n > 1):
                ok = False
                break
            try:
                lo, hi = Affine(rest, f.const).bounds(info.ranges)
            except KeyError:            # a loop whose trip count is not known when the kernel is generated
                ok = False
                break
            if lo < 0 or hi >= rowlen:
                ok = False
                break
            in_loop = in_loop or acc.loop_depth > 0
        if not ok or not in_loop:
            continue
        # rows padded to an odd number of 4-byte words: threads that read the same column of neighbouring rows hit
        # different banks
        padded = rowlen
        while (padded * itemsize) % 4 or ((padded * itemsize) // 4) % 2 == 0:
            padded += 1
            if itemsize >= 8:
                break                   # (8-byte elements: a two-way conflict is the best a row stride can do)
        bytes_ = (ROWS_BLOCK * padded * itemsize + 15) // 16 * 16
        if smem + bytes_ > ROWS_MAX_SMEM:
            continue
        staged.append((tensor, rowlen, padded, [a.node for a in accs], smem))
        smem += bytes_
    if not staged:
        return [], 0
    # Outputs whose every write lies in the writing worker's own row, unconditionally, the writes together covering
    # the whole row (``out[row, i] = ...`` in a loop over the row; ``out[row, 0] = ...`` followed by a loop from 1):
    # the rows are collected in shared memory and written out as one contiguous piece.
    writes = {}
    for acc in info.accesses:
        if acc.tensor.kind == 'output' and acc.is_write:
            writes.setdefault(id(acc.tensor), (acc.tensor, []))[1].append(acc)
    for tensor, accs in writes.values():
        size = tensor.size
        if size % W:
            continue
        rowlen = size // W
        itemsize = tensor.dtype.itemsize
        if rowlen < 2 or rowlen * itemsize > ROWS_MAX_ROW_BYTES:
            continue
        covered, ok = [], True
        for acc in accs:
            f = acc.form
            if f is None or f.mod is not None or acc.cond_depth > 0:
                ok = False
                break
            rest = {sym: c for sym, c in f.coefs.items() if sym[0] != 'p'}
            if any(f.coef(('p', d)) != rowlen * strides[d] for d, n in enumerate(shape) if n > 1):
                ok = False
                break
            # (a write covers the interval of its offsets only if the loop visits every value: step +-1)
            if len(rest) > 1 or any(abs(c) != 1 or abs(info.steps.get(sym, 0)) != 1 for sym, c in rest.items()):
                ok = False
                break
            try:
                lo, hi = Affine(rest, f.const).bounds(info.ranges)
            except KeyError:
                ok = False
                break
            if lo < 0 or hi >= rowlen:
                ok = False
                break
            covered.append((lo, hi))
        if not ok or not any(a.loop_depth > 0 for a in accs):
            continue
        reach = 0
        for lo, hi in sorted(covered):
            if lo > reach:
                break
            reach = max(reach, hi + 1)
        if reach < rowlen:
            continue                    # part of the row is never written: leave it alone
        padded = rowlen
        while (padded * itemsize) % 4 or ((padded * itemsize) // 4) % 2 == 0:
            padded += 1
            if itemsize >= 8:
                break
        bytes_ = (ROWS_BLOCK * padded * itemsize + 15) // 16 * 16
        if smem + bytes_ > ROWS_MAX_SMEM:
            continue
        staged.append((tensor, rowlen, padded, [a.node for a in accs], smem))
        smem += bytes_
    return staged, smem


def plan_tiling(kernel, info):
    """Accesses that walk memory along another workgroup axis than the innermost one (a transposed operand,
    ``out[i, j] = f(a[j, i], ...)``, or a transposed result, ``out[j, i] = f(a[i, j], ...)``).  Neighbouring
    workers of such an access are a whole stride apart, so a warp touches 32 sectors for 32 values.  Returns
    (axis, read slots, write slots, tile extents) when some accesses have coefficient 1 on workgroup axis ``axis`` and a
    larger stride on the innermost axis; read slots = [(tensor node, form, [read nodes])], write slots =
    [(tensor node, form, assign node)].  These accesses are staged through shared memory by tiles of
    up to TILE_WIDE x TILE_WIDE workers over (axis, innermost axis).  Only unconditional accesses outside loops whose
    address is provably inside the tensor for every worker qualify; a staged write must be the only statement
    that writes its tensor."""
    shape = kernel.workgroup_shape
    rank = len(shape)
    last = rank - 1
    if rank < 2 or shape[last] < TILE_EDGE:
        return None
    writers = {}
    for acc in info.accesses:
        if acc.is_write:
            writers[id(acc.tensor)] = writers.get(id(acc.tensor), 0) + 1
    reads, writes = {}, {}
    for acc in info.accesses:
        f = acc.form
        if f is None or f.mod is not None or acc.loop_depth > 0:
            continue
        if any(sym[0] == 'l' for sym in f.coefs):
            continue
        lo, hi = f.bounds(info.ranges)
        if lo < 0 or hi >= acc.tensor.size:
            continue            # (staging moves whole tiles: every worker's address must be valid)
        if abs(f.coef(('p', last))) < 2:
            continue
        if acc.is_write:
            if acc.tensor.kind != 'output' or acc.cond_depth > 0 or writers[id(acc.tensor)] != 1:
                continue
            if not _is_injective(f, info.ranges):
                continue
        elif acc.tensor.kind != 'input':
            continue
        for d in range(last):
            if shape[d] >= TILE_EDGE and f.coef(('p', d)) == 1:
                if acc.is_write:
                    writes.setdefault(d, []).append((acc.tensor, f, acc.node))
                else:
                    slot = reads.setdefault(d, {}).setdefault((id(acc.tensor), f.key()), [acc.tensor, f, []])
                    slot[2].append(acc.node)
    if not reads and not writes:
        return None
    axis = max(sorted(set(reads) | set(writes)), key=lambda d: len(reads.get(d, {})) + len(writes.get(d, [])))
    wanted_writes = writes.get(axis, [])
    wanted_reads = list(reads.get(axis, {}).values())
    # the widest tiles whose staging buffers fit; narrower tiles rather than fewer staged accesses
    for wide in (True, False):
        tile_t, tile_l = _tile_edges(shape, axis, wide)
        read_slots, write_slots, used = [], [], 0
        for tensor, form, node in wanted_writes:
            need = tile_l * (tile_t + 1) * tensor.dtype.itemsize
            if used + need <= TILE_SMEM_LIMIT:
                write_slots.append((tensor, form, node))
                used += need
        for tensor, form, nodes in wanted_reads:
            need = tile_l * (tile_t + 1) * tensor.dtype.itemsize
            if used + need <= TILE_SMEM_LIMIT:
                read_slots.append((tensor, form, nodes))
                used += need
        if len(read_slots) + len(write_slots) == len(wanted_reads) + len(wanted_writes):
            break
    if not read_slots and not write_slots:
        return None
    return axis, read_slots, write_slots, tile_t, tile_l


def _address_expr(form, shape):
    """C expression (uint64) of an affine offset at the group's first worker, from ``p<d>`` position names."""
    terms = []
    if form.const:
        terms.append(str(form.const) + 'ull')
    for (kind, d), c in sorted(form.coefs.items()):
        terms.append('(uint64_t)p' + str(d) + ('' if c == 1 else ' * ' + str(c) + 'ull'))
    return ' + '.join(terms) if terms else '0ull'


def _emit_tile(kernel, info, name, params, widx_t, math='exact'):
    """The ``_tile`` kernel: (source lines, metadata) or (None, None) when the kernel has no transposed accesses.

    Per tile of up to 64 x 64 workers over (axis, innermost axis): threads that walk the axis along which the
    operand is contiguous bring the staged operands into shared memory; the body runs with consecutive threads on
    consecutive workers of the innermost axis and takes the staged values from shared memory (transposed, rows
    padded by one element against bank conflicts); staged results go through shared memory the other way round."""
    tiling = plan_tiling(kernel, info)
    if tiling is None:
        return None, None
    shape = kernel.workgroup_shape
    axis, slots, wslots, tt, tl = tiling
    rank = len(shape)
    last = rank - 1
    n_t, n_l = (shape[axis] + tt - 1) // tt, (shape[last] + tl - 1) // tl
    n_tiles = n_t * n_l
    for d in range(rank):
        if d not in (axis, last):
            n_tiles *= shape[d]
    pitch = '[' + str(tl) + '][' + str(tt + 1) + ']'
    l_rows, t_rows = BLOCK_THREADS // tt, BLOCK_THREADS // tl      # rows covered at once when moving / computing
    read_subst, write_subst = {}, {}
    decls, stage, unstage = [], [], []
    for si, (tensor, form, nodes) in enumerate(slots):
        decls.append('    __shared__ ' + ctype(tensor.dtype) + ' ovl_tile' + str(si) + pitch + ';')
        stage.append('ovl_tile' + str(si) + '[ovl_ml + ovl_r][ovl_mt] = in' + str(tensor.attr['io_index']) + '[' +
                     _address_expr(form, shape) + '];')
        for n in nodes:
            read_subst[id(n)] = 'ovl_tile' + str(si) + '[ovl_cl][ovl_ct + ovl_r]'
    for si, (tensor, form, node) in enumerate(wslots):
        decls.append('    __shared__ ' + ctype(tensor.dtype) + ' ovl_wtile' + str(si) + pitch + ';')
        write_subst[id(node)] = 'ovl_wtile' + str(si) + '[ovl_cl][ovl_ct + ovl_r] = %s;'
        unstage.append('out' + str(tensor.attr['io_index']) + '[' + _address_expr(form, shape) + '] = ovl_wtile' + str(si) +
                       '[ovl_ml + ovl_r][ovl_mt];')
    decode = ['uint64_t ovl_rem = ovl_t;',
              'const uint32_t ovl_l0 = (uint32_t)(ovl_rem % ' + str(n_l) + 'ull) * ' + str(tl) + 'u; ovl_rem /= ' + str(n_l) + 'ull;',
              'const uint32_t ovl_t0 = (uint32_t)(ovl_rem % ' + str(n_t) + 'ull) * ' + str(tt) + 'u; ovl_rem /= ' + str(n_t) + 'ull;']
    for d in range(rank - 1, -1, -1):
        if d not in (axis, last):
            decode.append('const uint32_t ovl_q' + str(d) + ' = (uint32_t)(ovl_rem % ' + str(shape[d]) + 'ull); ovl_rem /= ' +
                          str(shape[d]) + 'ull;')

    def coords(t_expr, l_expr, var):
        out = []
        for d in range(rank):
            v = t_expr if d == axis else (l_expr if d == last else 'ovl_q' + str(d))
            out.append('const uint32_t ' + var + str(d) + ' = ' + v + ';')
        return out

    def inside(var):
        return var + str(axis) + ' < ' + str(shape[axis]) + 'u && ' + var + str(last) + ' < ' + str(shape[last]) + 'u'

    def moving(statements, comment):
        # consecutive threads walk the staged axis: whole contiguous segments of the tensor per row of the tile
        return [i2 + comment, i2 + '#pragma unroll',
                i2 + 'for (uint32_t ovl_r = 0; ovl_r < ' + str(tl) + 'u; ovl_r += ' + str(l_rows) + 'u) {'] + \
            [i3 + l for l in coords('ovl_t0 + ovl_mt', 'ovl_l0 + ovl_ml + ovl_r', 'p')] + \
            [i3 + 'if (' + inside('p') + ') {'] + [i4 + l for l in statements] + [i3 + '}', i2 + '}', i2 + '__syncthreads();']

    strides = _strides(shape)
    widx = ' + '.join('(' + widx_t + ')w' + str(d) + ' * ' + str(strides[d]) + 'u' for d in range(rank))
    pos_text = 'const uint32_t position[' + str(rank) + '] = {' + ', '.join('w' + str(d) for d in range(rank)) + '};'
    em = BodyEmitter(kernel, 4, read_subst, write_subst, position_text=pos_text, math=math)
    em.block(kernel.body)
    i1, i2, i3, i4 = '    ', '        ', '            ', '                '
    src = ['extern "C" __global__ void __launch_bounds__(' + str(BLOCK_THREADS) + ') ' + name + '_tile(' + params + ') {'] + \
        decls + \
        [i1 + '// thread coordinates inside a tile when moving data (mt fastest) and when computing (cl fastest)',
         i1 + 'const uint32_t ovl_mt = threadIdx.x % ' + str(tt) + 'u, ovl_ml = threadIdx.x / ' + str(tt) + 'u;',
         i1 + 'const uint32_t ovl_cl = threadIdx.x % ' + str(tl) + 'u, ovl_ct = threadIdx.x / ' + str(tl) + 'u;',
         i1 + 'for (uint64_t ovl_t = blockIdx.x; ovl_t < ' + str(n_tiles) + 'ull; ovl_t += gridDim.x) {'] + \
        [i2 + l for l in decode]
    if slots:
        src += moving(stage, '// stage the operands read along axis ' + str(axis))
    src += [i2 + '#pragma unroll',
            i2 + 'for (uint32_t ovl_r = 0; ovl_r < ' + str(tt) + 'u; ovl_r += ' + str(t_rows) + 'u) {'] + \
        [i3 + l for l in coords('ovl_t0 + ovl_ct + ovl_r', 'ovl_l0 + ovl_cl', 'w')] + \
        [i3 + 'if (' + inside('w') + ') {',
         i4 + 'const ' + widx_t + ' worker_index = ' + widx + '; (void)worker_index;'] + \
        em.lines + [i3 + '}', i2 + '}', i2 + '__syncthreads();']
    if wslots:
        src += moving(unstage, '// write the results that are contiguous along axis ' + str(axis))
    src += [i1 + '}', '}', '']
    return src, {'symbol': name + '_tile', 'block': BLOCK_THREADS, 'tiles': n_tiles, 'axis': axis, 'staged': len(slots),
                 'staged_writes': len(wslots)}


def plan_column_walk(spec):
    """Columns per strip (32, 16, 8 or 4) for the one-launch column scan, or None when the tensor has too few
    columns to give every SM a strip of its own (the three streaming passes split the rows instead).  Wide strips
    move whole 128-byte lines per row; narrower ones are taken only as far as needed to get a strip per SM, and never
    below 32 bytes per row."""
    itemsize = spec.dtype.itemsize
    widths = [w for w in (32, 16, 8, 4) if w * itemsize >= 32]
    strips = lambda w: spec.outer * ((spec.inner + w - 1) // w)      # noqa: E731
    for w in widths:
        if strips(w) >= COL_WALK_MIN_STRIPS:
            tile_rows = (COL_BLOCK // 32) * (32 // w) * col_walk_rows(itemsize)
            return w if spec.n * 2 >= tile_rows else None
    return None


def col_walk_rows(itemsize):
    return COL_WALK_REGS // max(1, itemsize // 4)        # 32 rows of up to 4-byte elements, 16 rows of 8-byte ones


SHORT_SCAN_BLOCK = 128
SHORT_SCAN_MIN_ELEMENTS = 1 << 16


def _short_scan_lines(spec):
    """Lines that ``ovl::scan_lines_short`` takes: at most 128 whole vectors each, enough of
    them to be worth a launch of their own (``ovl::scan_short_line``)."""
    if spec.inner != 1:
        return False
    vec = max(1, min(4, 16 // spec.dtype.itemsize))
    lanes = spec.n // vec
    return spec.n % vec == 0 and 1 <= lanes <= 128 and spec.lines * spec.n >= SHORT_SCAN_MIN_ELEMENTS


RING_GRID = 148                      # blocks of a ring scan on the target device (one per SM)
RING_GROUPED_MIN_EFFICIENCY = 0.93


def ring_group_efficiency(grid, lines, tiles_per_line):
    """Share of the grid's block-time that does useful work when every line is scanned by a group of blocks of its own
    (``ovl::ring_group_size`` / ``ovl::ring_group_efficiency`` of the templates): groups of grid // lines blocks, at
    most one block per tile of a line; lines are dealt to the groups in rounds."""
    g = 1 if lines >= grid else grid // lines
    g = max(1, min(g, tiles_per_line))
    groups = grid // g
    rounds = (lines + groups - 1) // groups
    return lines / float(rounds * groups) * (groups * g) / float(grid)


def _reduce_across_workers(kernel, info, red):
    """Should the threads of a warp be neighbouring WORKERS of a reduction loop rather than neighbouring trips of one
    worker's loop?  Yes when the loop's reads are strided along the loop variable but contiguous along the innermost
    workgroup axis (column sums: ``acc += a[i, col]``): then neighbouring workers' reads coalesce and neighbouring
    trips' do not."""
    shape = kernel.workgroup_shape
    last = ('p', len(shape) - 1)
    sym = info.loop_vars.get(id(red.fastest_var))
    if sym is None or shape[-1] < 8:        # (rows of fewer than 32 bytes: no layout reads them well)
        return False
    in_loop = set(id(n) for n in iter_nodes(red.loop.body))
    along = across = False
    for acc in info.accesses:
        if id(acc.node) not in in_loop or acc.is_write or acc.tensor.kind != 'input':
            continue
        if acc.form is None or acc.form.mod is not None:
            return False
        step = abs(acc.form.coef(sym))
        per_worker = any(k[0] == 'p' and c != 0 for k, c in acc.form.coefs.items())
        if step == 1 and per_worker:
            along = True                # (a read every worker shares, `w[i]`, is a broadcast in either layout)
        elif step > 1 and acc.form.coef(last) == 1:
            across = True
    return across and not along


def emit_cuda(kernel, name, math='exact', pack=True):
    """Full ``.cu`` text for one kernel plus its launch metadata.

    Returns (source, meta) with meta = {'gen': {...}, 'vec': {...} or None}; each entry has the symbol name, the
    block size and the number of loop iterations the grid should cover.

    ``math``: 'exact' - CUDA's libm and IEEE division, results within an ulp or two of the reference's C++
    operator; 'tolerance' - fp32 division, exp, log, log10, sqrt and tanh from csrc/templates/ovl_fastmath.cuh (results within
    rtol 1e-5, division within 2 ulp), and vectorised bodies of pure fp32 arithmetic evaluated two workers at a
    time with packed instructions (:mod:`opveclib_b200.cuda_pack`).  Integer work, data movement, fp64 and
    scans are the same in both."""
    if math not in MATH_MODES:
        raise ValueError('math must be one of ' + ', '.join(MATH_MODES))
    info = analyze(kernel)
    shape = kernel.workgroup_shape
    W = kernel.num_workers
    widx_t = 'uint32_t' if W < 2 ** 31 else 'uint64_t'
    params = ', '.join(_params(kernel))
    src = ['// generated by opveclib_b200 (' + TEMPLATE_VERSION + ', math=' + math + ') for kernel ' + kernel.name,
           '#include "ovl_common.cuh"', '']
    if math == 'tolerance':
        src.insert(2, '#include "ovl_fastmath.cuh"')

    # ---- generic kernel
    pos_text = 'const uint32_t position[' + str(len(shape)) + '] = {' + \
        ', '.join(_position_values(shape, 'worker_index')) + '};'
    em = BodyEmitter(kernel, 2, position_text=pos_text, math=math)
    em.block(kernel.body)
    src += ['extern "C" __global__ void __launch_bounds__(' + str(BLOCK_THREADS) + ') ' + name + '_gen(' + params +
            ') {',
            '    const ' + widx_t + ' ovl_stride = (' + widx_t + ')gridDim.x * ' + str(BLOCK_THREADS) + 'u;',
            '    for (' + widx_t + ' worker_index = (' + widx_t + ')blockIdx.x * ' + str(BLOCK_THREADS) +
            'u + threadIdx.x; worker_index < ' + str(W) + 'ull; worker_index += ovl_stride) {'] + em.lines + \
           ['    }', '}', '']
    meta = {'gen': {'symbol': name + '_gen', 'block': BLOCK_THREADS, 'items': W}, 'vec': None, 'scan': None, 'red': None,
            'tile': None, 'rows': None}

    # ---- vectorised kernel
    plan = plan_vectorisation(kernel, info)
    if plan.usable:
        L = plan.lanes
        groups = W // L
        last = len(shape) - 1
        read_subst, write_subst = {}, {}
        pre, post = [], []
        aligned_tensors = set()
        for si, (tensor, form, mode, nodes) in enumerate(plan.read_slots):
            t = ctype(tensor.dtype)
            tname = 'in' + str(tensor.attr['io_index'])
            if mode == 'vec':
                pre.append('const ovl::Vec<' + t + ', ' + str(L) + '> rv' + str(si) + ' = ovl::load_vec<' + t + ', ' +
                           str(L) + '>(' + tname + ' + (' + _address_expr(form, shape) + '));')
                for n in nodes:
                    read_subst[id(n)] = 'rv' + str(si) + '.v[ovl_lane]'
                aligned_tensors.add(('in', tensor.attr['io_index']))
            else:
                pre.append('const ' + t + ' ru' + str(si) + ' = *(' + tname + ' + (' +
                           _address_expr(form, shape) + '));')
                for n in nodes:
                    read_subst[id(n)] = 'ru' + str(si)
        for si, (tensor, form, nodes, conditional) in enumerate(plan.write_slots):
            t = ctype(tensor.dtype)
            tname = 'out' + str(tensor.attr['io_index'])
            pre.append('ovl::Vec<' + t + ', ' + str(L) + '> wv' + str(si) + ';')
            if conditional:
                pre.append('#pragma unroll')
                pre.append('for (int i = 0; i < ' + str(L) + '; ++i) wv' + str(si) + '.v[i] = 0;')
            for n in nodes:
                write_subst[id(n)] = 'wv' + str(si) + '.v[ovl_lane] = %s;'
            post.append('ovl::store_vec<' + t + ', ' + str(L) + '>(' + tname + ' + (' + _address_expr(form, shape) +
                        '), wv' + str(si) + ');')
            aligned_tensors.add(('out', tensor.attr['io_index']))
        pvals = _position_values(shape, 'ovl_w0')
        pos_decl = ['const uint32_t p' + str(d) + ' = ' + v + ';' for d, v in enumerate(pvals)]
        ind = '        '
        pairs = cuda_pack.plan_pairs(kernel, plan) if (math == 'tolerance' and pack) else None
        if pairs is not None:
            # two workers per expression: packed fp32 arithmetic, branches as masks
            read_text, write_name, open_pair, close_pair = {}, {}, [], []
            for si, (tensor, form, mode, nodes) in enumerate(plan.read_slots):
                for n in nodes:
                    read_text[id(n)] = ('ovl::tol::make2(rv%d.v[2 * ovl_pair], rv%d.v[2 * ovl_pair + 1])' % (si, si)
                                        if mode == 'vec' else 'ovl::tol::splat(ru%d)' % si)
            for si, (tensor, form, nodes, conditional) in enumerate(plan.write_slots):
                open_pair.append('ovl::tol::f2 wp%d = ovl::tol::splat(0.0f);' % si)
                close_pair.append('wv%d.v[2 * ovl_pair] = wp%d.x; wv%d.v[2 * ovl_pair + 1] = wp%d.y;' % (si, si, si, si))
                for n in nodes:
                    write_name[id(n)] = 'wp%d' % si
            em = cuda_pack.PairEmitter(kernel, 3, pairs, read_text, write_name, literal, _LIMITS)
            em.block(kernel.body)
            loop = [ind + '#pragma unroll', ind + 'for (int ovl_pair = 0; ovl_pair < ' + str(L // 2) + '; ++ovl_pair) {'] + \
                [ind + '    ' + l for l in open_pair] + em.lines + [ind + '    ' + l for l in close_pair] + [ind + '}']
        else:
            lane_pos = 'const uint32_t position[' + str(len(shape)) + '] = {' + ', '.join(
                ['p' + str(d) for d in range(last)] + ['p' + str(last) + ' + (uint32_t)ovl_lane']) + '};'
            em = BodyEmitter(kernel, 3, read_subst, write_subst, position_text=lane_pos, math=math)
            em.block(kernel.body)
            loop = [ind + '#pragma unroll', ind + 'for (int ovl_lane = 0; ovl_lane < ' + str(L) + '; ++ovl_lane) {',
                    ind + '    const ' + widx_t + ' worker_index = ovl_w0 + ovl_lane; (void)worker_index;'] + \
                em.lines + [ind + '}']
        src += ['extern "C" __global__ void __launch_bounds__(' + str(BLOCK_THREADS) + ') ' + name + '_vec(' +
                params + ') {',
                '    const ' + widx_t + ' ovl_stride = (' + widx_t + ')gridDim.x * ' + str(BLOCK_THREADS) + 'u;',
                '    for (' + widx_t + ' ovl_g = (' + widx_t + ')blockIdx.x * ' + str(BLOCK_THREADS) +
                'u + threadIdx.x; ovl_g < ' + str(groups) + 'ull; ovl_g += ovl_stride) {',
                ind + 'const ' + widx_t + ' ovl_w0 = ovl_g * ' + str(L) + 'u;'] + \
            [ind + l for l in pos_decl] + [ind + l for l in pre] + loop + [ind + l for l in post] + ['    }', '}', '']
        meta['vec'] = {'symbol': name + '_vec', 'block': BLOCK_THREADS, 'items': groups, 'lanes': L,
                       'aligned': sorted(aligned_tensors), 'paired': pairs is not None}
    # ---- transposed reads staged through shared memory
    tile_src, tile_meta = _emit_tile(kernel, info, name, params, widx_t, math)
    if tile_src is not None:
        src += tile_src
        meta['tile'] = tile_meta
    # ---- rows staged in shared memory (per-worker loops over the worker's own row of an input)
    staged, rows_smem = plan_row_staging(kernel, info)
    if staged:
        read_subst, rows_write_subst = {}, {}
        head, stage, unstage = [], [], []
        for k, (tensor, rowlen, padded, nodes, offset) in enumerate(staged):
            t = ctype(tensor.dtype)
            head.append('    ' + t + '* const ovl_row' + str(k) + ' = reinterpret_cast<' + t + '*>(ovl_rows_smem + ' +
                        str(offset) + ');')
            if tensor.kind == 'output':
                tname = 'out' + str(tensor.attr['io_index'])
                stage.append('        const uint64_t ovl_first' + str(k) + ' = (uint64_t)ovl_w0 * ' + str(rowlen) + 'ull;')
                unstage += ['        #pragma unroll 4',
                            '        for (uint32_t ovl_e = threadIdx.x; ovl_e < ovl_live * ' + str(rowlen) + 'u; ovl_e += ' +
                            str(ROWS_BLOCK) + 'u)',
                            '            ' + tname + '[ovl_first' + str(k) + ' + ovl_e] = ovl_row' + str(k) + '[ovl_e + (ovl_e / ' +
                            str(rowlen) + 'u) * ' + str(padded - rowlen) + 'u];']
                for n in nodes:
                    rows_write_subst[id(n)] = 'ovl_row' + str(k) + '[(uint32_t)({index} - ovl_first' + str(k) + \
                        ') + threadIdx.x * ' + str(padded - rowlen) + 'u] = %s;'
                continue
            tname = 'in' + str(tensor.attr['io_index'])
            slot = 'ovl_row' + str(k) + '[ovl_e + (ovl_e / ' + str(rowlen) + 'u) * ' + str(padded - rowlen) + 'u]'
            source = tname + '[ovl_first' + str(k) + ' + ovl_e]'
            # 4- and 8-byte elements travel by asynchronous copies (no registers in between, any number in flight)
            if tensor.dtype.itemsize in (4, 8):
                move = 'ovl::cp_async_vec<' + str(tensor.dtype.itemsize) + '>(&' + slot + ', &' + source + ');'
            else:
                move = slot + ' = ' + source + ';'
            stage += ['        const uint64_t ovl_first' + str(k) + ' = (uint64_t)ovl_w0 * ' + str(rowlen) + 'ull;',
                      '        #pragma unroll 4',
                      '        for (uint32_t ovl_e = threadIdx.x; ovl_e < ovl_live * ' + str(rowlen) + 'u; ovl_e += ' +
                      str(ROWS_BLOCK) + 'u)',
                      '            ' + move]
            for n in nodes:
                read_subst[id(n)] = 'ovl_row' + str(k) + '[(uint32_t)({index} - ovl_first' + str(k) + ') + threadIdx.x * ' + \
                    str(padded - rowlen) + 'u]'
        em = BodyEmitter(kernel, 3, read_subst, rows_write_subst, position_text=pos_text, math=math)
        em.block(kernel.body)
        if unstage:
            unstage = ['        __syncthreads();        // every row of the block is complete'] + unstage
        src += ['extern "C" __global__ void __launch_bounds__(' + str(ROWS_BLOCK) + ') ' + name + '_rows(' + params + ') {',
                '    extern __shared__ __align__(16) unsigned char ovl_rows_smem[];'] + head + \
               ['    for (' + widx_t + ' ovl_w0 = (' + widx_t + ')blockIdx.x * ' + str(ROWS_BLOCK) + 'u; ovl_w0 < ' + str(W) +
                'ull; ovl_w0 += (' + widx_t + ')gridDim.x * ' + str(ROWS_BLOCK) + 'u) {',
                '        // the rows of this block\'s workers are one contiguous piece of each staged tensor',
                '        const uint32_t ovl_live = (' + str(W) + 'ull - ovl_w0 < ' + str(ROWS_BLOCK) + 'u) ? (uint32_t)(' +
                str(W) + 'ull - ovl_w0) : ' + str(ROWS_BLOCK) + 'u;'] + stage + \
               ['        ovl::cp_async_commit();',
                '        ovl::cp_async_wait_all();',
                '        __syncthreads();',
                '        if (threadIdx.x < ovl_live) {',
                '            const ' + widx_t + ' worker_index = ovl_w0 + threadIdx.x;'] + em.lines + \
               ['        }'] + unstage + \
               ['        __syncthreads();        // the next round overwrites the rows',
                '    }', '}', '']
        meta['rows'] = {'symbol': name + '_rows', 'block': ROWS_BLOCK, 'items': W, 'smem': rows_smem,
                        'staged': [[tensor.attr['io_index'], rowlen] for tensor, rowlen, _, _, _ in staged
                                   if tensor.kind == 'input'],
                        'staged_outputs': [[tensor.attr['io_index'], rowlen] for tensor, rowlen, _, _, _ in staged
                                           if tensor.kind == 'output']}
    # ---- cooperative reduction loop
    red = patterns.match_reduce(kernel, info)
    if red is not None and red.inner is not None and _reduce_across_workers(kernel, info, red):
        red = None          # a nest whose reads are contiguous across workers: the generic kernel reads it coalesced
    if red is not None:
        src.insert(2, '#include "ovl_reduce.cuh"')
        across = _reduce_across_workers(kernel, info, red) and os.environ.get('OVL_RED_LAYOUT') != 'along'
        group = REDUCE_BLOCK if (red.n >= REDUCE_BLOCK_TRIPS and W < REDUCE_FEW_WORKERS) else 32
        red_block = REDUCE_BLOCK
        if across:
            # 32 neighbouring workers per block, the loop cut into as many slices as the block has warps: 8, or 32
            # when there are too few workers to fill the device with 256-thread blocks
            if (W + 31) // 32 < REDUCE_ACROSS_WIDE_BELOW and red.n >= 1024:
                red_block = 1024
            group = red_block // 32
        per_block = red_block // group
        top = kernel.body.nodes
        at = [i for i, x in enumerate(top) if x is red.loop][0]
        em = BodyEmitter(kernel, 2, position_text=pos_text, math=math)
        for node in top[:at]:
            em.node(node)
        acc_t = ctype(red.acc.dtype)
        opname = 'ovl::OpAdd' if red.op == 'add' else 'ovl::OpMul'
        ivar = em.name(red.loop.args[0])
        ivar_t = ctype(red.loop.args[0].dtype)
        if red.inner is not None:
            # a nest of two loops runs as one loop over its trips; the loop variables are derived from the trip
            ivar, ivar_t = 'ovl_trip', 'uint64_t'
            em.put('uint64_t ovl_trip;')
        # few workers with long loops: the loop of a worker is cut into slices that different blocks fold
        if across:
            split = (W + 31) // 32 <= REDUCE_SPLIT_MAX_WORKERS // 2 and red.n >= REDUCE_SPLIT_MIN_TRIPS // 2
        else:
            split = group == REDUCE_BLOCK and W <= REDUCE_SPLIT_MAX_WORKERS and red.n >= REDUCE_SPLIT_MIN_TRIPS
        split = split and os.environ.get('OVL_RED_SPLIT') != 'off'
        em.put(acc_t + ' ovl_partial = ' + opname + '::identity<' + acc_t + '>();')
        em.put('#pragma unroll ' + ('8' if across else '4'))
        if split:
            em.put('for(' + ivar + ' = (' + ivar_t + ')(ovl_lo + ovl_member); ' + ivar + ' < (' + ivar_t + ')ovl_hi; ' +
                   ivar + ' += ' + str(group) + '){')
        else:
            em.put('for(' + ivar + ' = ovl_member; ' + ivar + ' < ' + str(red.n) + '; ' + ivar + ' += ' + str(group) + '){')
        em.depth += 1

        def fold_body(nodes):
            for node in nodes:
                if node is red.update:
                    em.put('ovl_partial = ' + opname + '::apply<' + acc_t + '>(ovl_partial, ' + em.name(red.term) + ');')
                else:
                    em.node(node)
        if red.inner is None:
            fold_body(red.loop.body.nodes)
        else:
            outer_var, inner_var = red.loop.args[0], red.inner.args[0]
            em.put(em.name(outer_var) + ' = (' + ctype(outer_var.dtype) + ')(ovl_trip / ' + str(red.n_inner) + 'ull);')
            for node in red.loop.body.nodes:
                if node is red.inner:
                    em.put(em.name(inner_var) + ' = (' + ctype(inner_var.dtype) + ')(ovl_trip % ' + str(red.n_inner) + 'ull);')
                    fold_body(red.inner.body.nodes)
                else:
                    em.node(node)
        em.depth -= 1
        em.put('}')
        fold_cols = ['ovl_red_cols[ovl_member][ovl_tx] = %s;', '__syncthreads();']
        if across and split:
            col_groups = (W + 31) // 32
            slice_min = REDUCE_SPLIT_SLICE // 4
            max_splits = max(1, min(REDUCE_SPLIT_MAX, red.n // slice_min))
            counter_bytes = SCAN_HEADER_BYTES + (4 * col_groups + 15) // 16 * 16
            acc_size = red.acc.dtype.itemsize
            fold_all = ['    ' + acc_t + ' ovl_all = ovl_red_cols[0][ovl_tx];', '    #pragma unroll',
                        '    for (int ovl_s = 1; ovl_s < ' + str(group) + '; ++ovl_s) ovl_all = ' + opname + '::apply<' +
                        acc_t + '>(ovl_all, ovl_red_cols[ovl_s][ovl_tx]);']
            # every block leaves the totals of its slice (32 columns) in the column group's row of partial results;
            # the block that delivers the last slice folds the row in slice order and finishes the 32 workers
            for line in [fold_cols[0] % 'ovl_partial', fold_cols[1],
                         acc_t + '* const ovl_row = reinterpret_cast<' + acc_t + '*>(reinterpret_cast<char*>(scratch) + ' +
                         str(counter_bytes) + ') + (uint64_t)ovl_group_index * ' + str(max_splits * 32) + 'ull;',
                         'if (ovl_member == 0) {'] + fold_all + [
                         '    ovl_row[ovl_split * 32u + ovl_tx] = ovl_all;', '    __threadfence();', '}',
                         '__syncthreads();',
                         'if (threadIdx.x == 0) ovl_last = atomicAdd(reinterpret_cast<uint32_t*>(reinterpret_cast<char*>('
                         'scratch) + ' + str(SCAN_HEADER_BYTES) + ') + ovl_group_index, 1u) == ovl_splits - 1u;',
                         '__syncthreads();', 'if (!ovl_last) return;', '__threadfence();',
                         acc_t + ' ovl_fold = ' + opname + '::identity<' + acc_t + '>();',
                         'for (uint32_t ovl_s = ovl_member; ovl_s < ovl_splits; ovl_s += ' + str(group) + 'u) ovl_fold = ' +
                         opname + '::apply<' + acc_t + '>(ovl_fold, *(volatile ' + acc_t + '*)&ovl_row[ovl_s * 32u + ovl_tx]);',
                         fold_cols[0] % 'ovl_fold', fold_cols[1], 'if (ovl_member == 0) {'] + fold_all:
                em.put(line)
            em.depth += 1
            em.put(em.name(red.acc) + ' = ' + opname + '::apply<' + acc_t + '>(' + em.name(red.acc) + ', ovl_all);')
            em.put('if (ovl_live) {')
            em.depth += 1
            for node in top[at + 1:]:
                em.node(node)
            em.depth -= 1
            em.put('}')
            em.depth -= 1
            em.put('}')
            slice_len = '((' + str(red.n) + 'ull + ovl_splits - 1u) / ovl_splits + ' + str(group - 1) + 'ull) / ' + \
                str(group) + 'ull * ' + str(group) + 'ull'
            src += ['extern "C" __global__ void __launch_bounds__(' + str(red_block) + ') ' + name + '_red(' + params +
                    ', void* scratch) {',
                    '    __shared__ ' + acc_t + ' ovl_red_cols[' + str(group) + '][32];',
                    '    __shared__ bool ovl_last;',
                    '    const uint32_t ovl_tx = threadIdx.x & 31u, ovl_member = threadIdx.x >> 5;',
                    '    // grid = groups of 32 workers x slices of the loop',
                    '    const uint32_t ovl_splits = gridDim.x / ' + str(col_groups) + 'u;',
                    '    const uint32_t ovl_group_index = blockIdx.x / ovl_splits, ovl_split = blockIdx.x % ovl_splits;',
                    '    const uint64_t ovl_len = ' + slice_len + ';',
                    '    const uint64_t ovl_lo = (uint64_t)ovl_split * ovl_len;',
                    '    const uint64_t ovl_hi = ovl_lo + ovl_len < ' + str(red.n) + 'ull ? ovl_lo + ovl_len : ' + str(red.n) + 'ull;',
                    '    const ' + widx_t + ' ovl_base = (' + widx_t + ')ovl_group_index * 32u;',
                    '    const bool ovl_live = ovl_base + ovl_tx < ' + str(W) + 'ull;',
                    '    const ' + widx_t + ' worker_index = ovl_live ? ovl_base + ovl_tx : (' + widx_t + ')' + str(W - 1) + 'ull;',
                    '    {'] + em.lines + ['    }', '}', '']
            meta['red'] = {'symbol': name + '_red', 'block': red_block, 'workers_per_block': 32, 'items': W,
                           'group': group, 'trips': red.n, 'op': red.op, 'layout': 'across',
                           'split': {'max': max_splits, 'slice': slice_min, 'units': col_groups,
                                     'scratch_bytes': counter_bytes + col_groups * max_splits * 32 * acc_size,
                                     'zero_bytes': counter_bytes}}
        elif across:
            em.put('ovl_red_cols[ovl_member][ovl_tx] = ovl_partial;')
            em.put('__syncthreads();')
            em.put('if (ovl_member == 0) {')
            em.depth += 1
            em.put(acc_t + ' ovl_all = ovl_red_cols[0][ovl_tx];')
            em.put('#pragma unroll')
            em.put('for (int ovl_s = 1; ovl_s < ' + str(group) + '; ++ovl_s) ovl_all = ' + opname + '::apply<' + acc_t +
                   '>(ovl_all, ovl_red_cols[ovl_s][ovl_tx]);')
            em.put(em.name(red.acc) + ' = ' + opname + '::apply<' + acc_t + '>(' + em.name(red.acc) + ', ovl_all);')
            em.put('if (ovl_live) {')
            em.depth += 1
            for node in top[at + 1:]:
                em.node(node)
            em.depth -= 1
            em.put('}')
            em.depth -= 1
            em.put('}')
            em.put('__syncthreads();')
            # neighbouring threads are neighbouring workers (their reads coalesce); the warps of a block share the loop
            src += ['extern "C" __global__ void __launch_bounds__(' + str(red_block) + ') ' + name + '_red(' + params + ') {',
                    '    __shared__ ' + acc_t + ' ovl_red_cols[' + str(group) + '][32];',
                    '    const uint32_t ovl_tx = threadIdx.x & 31u, ovl_member = threadIdx.x >> 5;',
                    '    for (' + widx_t + ' ovl_base = (' + widx_t + ')blockIdx.x * 32u; ovl_base < ' + str(W) +
                    'ull; ovl_base += (' + widx_t + ')gridDim.x * 32u) {',
                    '        const bool ovl_live = ovl_base + ovl_tx < ' + str(W) + 'ull;',
                    '        // (threads past the last worker repeat it, so that every thread reaches the barriers)',
                    '        const ' + widx_t + ' worker_index = ovl_live ? ovl_base + ovl_tx : (' + widx_t + ')' + str(W - 1) +
                    'ull;'] + em.lines + ['    }', '}', '']
            meta['red'] = {'symbol': name + '_red', 'block': red_block, 'workers_per_block': 32, 'items': W,
                           'group': group, 'trips': red.n, 'op': red.op, 'layout': 'across'}
    if red is not None and split and not across:
        max_splits = max(1, min(REDUCE_SPLIT_MAX, red.n // REDUCE_SPLIT_SLICE))
        # scratch: 16-byte header (the status word every kernel with scratch has; stays 0), one counter per worker,
        # then the rows of partial results
        counter_bytes = SCAN_HEADER_BYTES + (4 * W + 15) // 16 * 16
        acc_size = red.acc.dtype.itemsize
        # the slice's result goes to the worker's row of partial results; the block that delivers the last one folds
        # the row in slice order (members take slices m, m + 256, ...; then the usual combination) and finishes the
        # worker.  Which block that is does not matter to the result.
        em.put('const ' + acc_t + ' ovl_slice = ovl::group_reduce<' + acc_t + ', ' + opname + ', ' + str(group) +
               '>(ovl_partial, ovl_red_smem);')
        em.put('uint32_t* const ovl_count = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(scratch) + ' +
               str(SCAN_HEADER_BYTES) + ') + worker_index;')
        em.put(acc_t + '* const ovl_row = reinterpret_cast<' + acc_t + '*>(reinterpret_cast<char*>(scratch) + ' +
               str(counter_bytes) + ') + (uint64_t)worker_index * ' + str(max_splits) + 'ull;')
        em.put('if (threadIdx.x == 0) {')
        em.put('    ovl_row[ovl_split] = ovl_slice;')
        em.put('    __threadfence();')
        em.put('    ovl_last = atomicAdd(ovl_count, 1u) == ovl_splits - 1u;')
        em.put('}')
        em.put('__syncthreads();')
        em.put('if (!ovl_last) return;')
        em.put('__threadfence();')
        em.put(acc_t + ' ovl_fold = ' + opname + '::identity<' + acc_t + '>();')
        em.put('for (uint32_t ovl_s = ovl_member; ovl_s < ovl_splits; ovl_s += ' + str(group) + 'u) ovl_fold = ' + opname +
               '::apply<' + acc_t + '>(ovl_fold, *(volatile ' + acc_t + '*)&ovl_row[ovl_s]);')
        em.put(em.name(red.acc) + ' = ' + opname + '::apply<' + acc_t + '>(' + em.name(red.acc) + ', ovl::group_reduce<' +
               acc_t + ', ' + opname + ', ' + str(group) + '>(ovl_fold, ovl_red_smem));')
        em.put('if (ovl_member == 0) {')
        em.depth += 1
        for node in top[at + 1:]:
            em.node(node)
        em.depth -= 1
        em.put('}')
        slice_len = '((' + str(red.n) + 'ull + ovl_splits - 1u) / ovl_splits + ' + str(group - 1) + 'ull) / ' + \
            str(group) + 'ull * ' + str(group) + 'ull'
        src += ['extern "C" __global__ void __launch_bounds__(' + str(REDUCE_BLOCK) + ') ' + name + '_red(' + params +
                ', void* scratch) {',
                '    __shared__ ' + acc_t + ' ovl_red_smem[' + str(REDUCE_BLOCK // 32) + '];',
                '    __shared__ bool ovl_last;',
                '    const uint32_t ovl_member = threadIdx.x;',
                '    // grid = workers x slices: block b folds slice b % slices of worker b / slices',
                '    const uint32_t ovl_splits = gridDim.x / ' + str(W) + 'u;',
                '    const ' + widx_t + ' worker_index = blockIdx.x / ovl_splits;',
                '    const uint32_t ovl_split = blockIdx.x % ovl_splits;',
                '    const uint64_t ovl_len = ' + slice_len + ';',
                '    const uint64_t ovl_lo = (uint64_t)ovl_split * ovl_len;',
                '    const uint64_t ovl_hi = ovl_lo + ovl_len < ' + str(red.n) + 'ull ? ovl_lo + ovl_len : ' + str(red.n) + 'ull;',
                '    {'] + em.lines + ['    }', '}', '']
        meta['red'] = {'symbol': name + '_red', 'block': REDUCE_BLOCK, 'workers_per_block': 1, 'items': W,
                       'group': group, 'trips': red.n, 'op': red.op, 'layout': 'along',
                       'split': {'max': max_splits, 'slice': REDUCE_SPLIT_SLICE, 'units': W,
                                 'scratch_bytes': counter_bytes + W * max_splits * acc_size,
                                 'zero_bytes': counter_bytes}}
    elif red is not None and not across:
        em.put(em.name(red.acc) + ' = ' + opname + '::apply<' + acc_t + '>(' + em.name(red.acc) + ', ovl::group_reduce<' +
               acc_t + ', ' + opname + ', ' + str(group) + '>(ovl_partial, ovl_red_smem));')
        em.put('if (ovl_member == 0) {')
        em.depth += 1
        for node in top[at + 1:]:
            em.node(node)
        em.depth -= 1
        em.put('}')
        src += ['extern "C" __global__ void __launch_bounds__(' + str(REDUCE_BLOCK) + ') ' + name + '_red(' + params + ') {',
                '    __shared__ ' + acc_t + ' ovl_red_smem[' + str(REDUCE_BLOCK // 32) + '];',
                '    const uint32_t ovl_member = threadIdx.x % ' + str(group) + 'u;',
                '    const ' + widx_t + ' ovl_stride = (' + widx_t + ')gridDim.x * ' + str(per_block) + 'u;',
                '    for (' + widx_t + ' worker_index = (' + widx_t + ')blockIdx.x * ' + str(per_block) + 'u + threadIdx.x / ' +
                str(group) + 'u; worker_index < ' + str(W) + 'ull; worker_index += ovl_stride) {'] + em.lines + \
               ['    }', '}', '']
        meta['red'] = {'symbol': name + '_red', 'block': REDUCE_BLOCK, 'workers_per_block': per_block, 'items': W,
                       'group': group, 'trips': red.n, 'op': red.op, 'layout': 'along'}
    # ---- cooperative scan
    spec = patterns.match_scan(kernel, info)
    if spec is not None and spec.inner > 1:
        # scan along a non-contiguous axis: warps walk down strips of columns, three streaming passes
        if spec.n >= patterns.COLSCAN_MIN_AXIS:
            src.insert(2, '#include "ovl_colscan.cuh"')
            t = ctype(spec.dtype)
            acc = 'double' if spec.dtype.is_float else t
            acc_size = 8 if spec.dtype.is_float else spec.dtype.itemsize
            vec = max(1, 16 // spec.dtype.itemsize)
            op = 'ovl::OpAdd' if spec.op == 'add' else 'ovl::OpMul'
            chunks = (spec.n + COL_ROWS - 1) // COL_ROWS
            can_align = spec.inner % vec == 0
            agg_ptr = '(' + acc + '*)((char*)scratch + ' + str(SCAN_HEADER_BYTES) + ')'
            dims = str(spec.outer) + 'ull, ' + str(spec.n) + 'ull, ' + str(spec.inner) + 'ull'
            tiles = {}
            for suffix, v in [('u', 1)] + ([('', vec)] if can_align else []):
                strips = (spec.inner + 32 * v - 1) // (32 * v)
                tiles[suffix] = spec.outer * chunks * strips
                src += ['extern "C" __global__ void __launch_bounds__(' + str(COL_BLOCK) + ') ' + name + '_cagg' + suffix +
                        '(const ' + t + '* __restrict__ in0, void* scratch) {',
                        '    ovl::col_tiles<' + t + ', ' + acc + ', ' + op + ', ' + str(v) + ', false>(in0, nullptr, ' + agg_ptr +
                        ', ' + dims + ');', '}', '',
                        'extern "C" __global__ void __launch_bounds__(' + str(COL_BLOCK) + ') ' + name + '_cscan' + suffix +
                        '(const ' + t + '* __restrict__ in0, ' + t + '* __restrict__ out0, void* scratch) {',
                        '    ovl::col_tiles<' + t + ', ' + acc + ', ' + op + ', ' + str(v) + ', true>(in0, out0, ' + agg_ptr +
                        ', ' + dims + ');', '}', '']
            src += ['extern "C" __global__ void __launch_bounds__(' + str(COL_BLOCK) + ') ' + name + '_cpfx(void* scratch) {',
                    '    ovl::col_prefixes<' + acc + ', ' + op + '>(' + agg_ptr + ', ' + dims + ');', '}', '']
            walk = None
            width = plan_column_walk(spec)
            if width is not None:
                # enough columns: one block walks down all rows of a strip of `width` columns, one launch
                src += ['extern "C" __global__ void __launch_bounds__(' + str(COL_BLOCK) + ', 2) ' + name +
                        '_cwalk(const ' + t + '* __restrict__ in0, ' + t + '* __restrict__ out0) {',
                        '    ovl::col_walk<' + t + ', ' + acc + ', ' + op + ', ' + str(width) + ', ' + str(COL_BLOCK // 32) +
                        ', ' + str(col_walk_rows(spec.dtype.itemsize)) + '>(in0, out0, ' + dims + ');', '}', '']
                walk = {'symbol': name + '_cwalk', 'block': COL_BLOCK, 'width': width,
                        'strips': spec.outer * ((spec.inner + width - 1) // width)}
            meta['scan'] = {'name': name, 'strided': True, 'aligned_variant': bool(can_align), 'block': COL_BLOCK, 'walk': walk,
                            'tiles': tiles, 'columns': spec.outer * spec.inner,
                            'scratch_bytes': SCAN_HEADER_BYTES + spec.outer * chunks * spec.inner * acc_size,
                            'zero_bytes': SCAN_HEADER_BYTES, 'align_bytes': 16, 'lines': spec.lines, 'n': spec.n,
                            'outer': spec.outer, 'inner': spec.inner, 'op': spec.op, 'ring': None}
    elif spec is not None and (spec.n >= patterns.SCAN_MIN_AXIS or _short_scan_lines(spec) or
                               (spec.lines >= WARP_SCAN_MIN_LINES and spec.n >= WARP_SCAN_MIN_AXIS and
                                (spec.n * spec.dtype.itemsize) % 16 == 0)):
        src.insert(2, '#include "ovl_scan.cuh"')
        t = ctype(spec.dtype)
        acc = 'double' if spec.dtype.is_float else t
        acc_size = 8 if spec.dtype.is_float else spec.dtype.itemsize
        vec = max(1, min(4, 16 // spec.dtype.itemsize))
        tile = SCAN_BLOCK * SCAN_VPT * vec
        multi = spec.n > tile                       # several tiles per line: three passes
        tpl = (spec.n + tile - 1) // tile if multi else 1
        tiles = tpl * spec.lines
        scratch = SCAN_HEADER_BYTES + tiles * 16     # one fp64 / two tagged words per tile
        op = 'ovl::OpAdd' if spec.op == 'add' else 'ovl::OpMul'
        can_align = spec.lines == 1 or spec.n % vec == 0
        agg_ptr = '(' + acc + '*)((char*)scratch + ' + str(SCAN_HEADER_BYTES) + ')'
        mode = 'ovl::kScanPrefixed' if multi else 'ovl::kScanOneTile'
        for suffix, aligned in [('u', 'false')] + ([('', 'true')] if can_align else []):
            src += ['extern "C" __global__ void __launch_bounds__(' + str(SCAN_BLOCK) + ', 2) ' + name + '_scan' + suffix +
                    '(const ' + t + '* __restrict__ in0, ' + t + '* __restrict__ out0, void* scratch) {',
                    '    ovl::scan_lines<' + t + ', ' + acc + ', ' + op + ', ' + str(vec) + ', ' + aligned + ', false, ' +
                    mode + '>(in0, out0, nullptr, ' + str(spec.lines) + 'ull, ' + str(spec.n) + 'ull, scratch);',
                    '}', '']
            if multi:
                src += ['extern "C" __global__ void __launch_bounds__(' + str(SCAN_BLOCK) + ', 2) ' + name + '_agg' +
                        suffix + '(const ' + t + '* __restrict__ in0, void* scratch) {',
                        '    ovl::tile_aggregates<' + t + ', ' + acc + ', ' + op + ', ' + str(vec) + ', ' + aligned +
                        '>(in0, ' + str(spec.lines) + 'ull, ' + str(spec.n) + 'ull, ' + agg_ptr + ');',
                        '}', '']
        if multi:
            src += ['extern "C" __global__ void __launch_bounds__(' + str(SCAN_BLOCK) + ') ' + name +
                    '_pfx(void* scratch) {',
                    '    ovl::scan_aggregates<' + acc + ', ' + op + ', false, true>(' + agg_ptr + ', ' + str(spec.lines) +
                    'ull, ' + str(tpl) + 'ull, nullptr, nullptr);',
                    '}', '']
        warp = None
        if _short_scan_lines(spec):
            # short lines: the tensor streamed as a flat array of vectors, as many whole lines per warp as fit
            src += ['extern "C" __global__ void __launch_bounds__(' + str(SHORT_SCAN_BLOCK) + ') ' + name +
                    '_wscan(const ' + t + '* __restrict__ in0, ' + t + '* __restrict__ out0) {',
                    '    ovl::scan_lines_short<' + t + ', ' + acc + ', ' + op + ', ' + str(vec) + '>(in0, out0, ' +
                    str(spec.lines) + 'ull, ' + str(spec.n) + 'u);',
                    '}', '']
            per_chunk = 128 // (spec.n // vec)       # whole lines per warp and step
            warp = {'symbol': name + '_wscan', 'block': SHORT_SCAN_BLOCK, 'flat_vectors': spec.lines * (spec.n // vec),
                    'chunks': (spec.lines + per_chunk - 1) // per_chunk}
        elif spec.lines >= WARP_SCAN_MIN_LINES and (spec.n * spec.dtype.itemsize) % 16 == 0:
            # thousands of lines: a warp per line, nothing shared between warps
            src += ['extern "C" __global__ void __launch_bounds__(' + str(WARP_SCAN_BLOCK) + ') ' + name +
                    '_wscan(const ' + t + '* __restrict__ in0, ' + t + '* __restrict__ out0) {',
                    '    ovl::scan_lines_warp<' + t + ', ' + acc + ', ' + op + ', ' + str(vec) + '>(in0, out0, ' +
                    str(spec.lines) + 'ull, ' + str(spec.n) + 'ull);',
                    '}', '']
            warp = {'symbol': name + '_wscan', 'block': WARP_SCAN_BLOCK}
        ring = None
        # (bulk copies need every line to start on a 16-byte boundary)
        if multi and can_align and (spec.lines == 1 or (spec.n * spec.dtype.itemsize) % 16 == 0):
            # long lines, pointers aligned: a single cooperative launch that moves every element once
            # several lines: each scanned by a group of blocks of its own when that keeps a B200's grid busy (the same
            # rule as ovl::ring_group_efficiency), otherwise waves that cross line ends
            layout = 'false, false'
            if spec.lines > 1:
                grouped = ring_group_efficiency(RING_GRID, spec.lines, tpl) >= RING_GROUPED_MIN_EFFICIENCY
                layout = 'false, false, false, false, true' if grouped else 'false, true'
            src += ['extern "C" __global__ void __launch_bounds__(' + str(RING_THREADS) + ', 1) ' + name +
                    '_ring(const ' + t + '* __restrict__ in0, ' + t + '* __restrict__ out0, void* scratch) {',
                    '    ovl::scan_ring<' + t + ', ' + acc + ', ' + op + ', ' + str(vec) + ', ' + layout +
                    '>(in0, out0, nullptr, ' + str(spec.lines) + 'ull, ' + str(spec.n) + 'ull, scratch);',
                    '}', '']
            ring = {'symbol': name + '_ring', 'block': RING_THREADS, 'max_grid': RING_MAX_GRID,
                    'layout': 'single' if spec.lines == 1 else ('grouped' if layout.endswith('true') and layout.count(',') > 1
                                                                 else 'waves'),
                    'smem': RING_SLOTS * tile * spec.dtype.itemsize + RING_CTL_BYTES,
                    'zero_bytes': SCAN_HEADER_BYTES + tiles * 16}
        meta['scan'] = {'name': name, 'aligned_variant': bool(can_align), 'three_pass': bool(multi), 'ring': ring,
                        'warp': warp, 'short': spec.n < patterns.SCAN_MIN_AXIS,
                        'block': SCAN_BLOCK, 'tiles': tiles, 'scratch_bytes': scratch, 'zero_bytes': SCAN_HEADER_BYTES,
                        'blocks_per_sm': 2, 'align_bytes': vec * spec.dtype.itemsize, 'lines': spec.lines, 'n': spec.n,
                        'op': spec.op}
    return '\n'.join(src), meta
