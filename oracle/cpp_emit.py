"""TEST INFRASTRUCTURE - CPU oracle, never part of the product path.

Restates the reference's C++ code generator for one operator: given a traced kernel it emits the C++ worker
function the reference would emit (``ExpressionDAG.generate``, opveclib/expression.py:522-593 and 649-670) -
one statement per expression, in trace order, each with the expression's own C type, wrapped in the
per-thread loop ``for worker_index in [thread*block, min((thread+1)*block, W))``.  Statement forms follow the
per-node ``gen_c`` methods cited beside each emitter below.  Only tests/, the smoke check and the benchmark's
CPU-baseline leg may import this module.

Parity of this restatement is pinned against outputs of the reference's own generator and C++ operators run in
the development container (tests/golden/*.npz, produced by tests/golden/make_golden.py).
"""
import math

from opveclib_b200 import expr as E

# opveclib/expression.py:1430-1456
_UNARY_F32 = {'acos': 'acosf', 'asin': 'asinf', 'atan': 'atanf', 'cos': 'cosf', 'cosh': 'coshf', 'sin': 'sinf',
              'sinh': 'sinhf', 'tan': 'tanf', 'tanh': 'tanhf', 'exp': 'expf', 'log': 'logf', 'log10': 'log10f',
              'sqrt': 'sqrtf', 'ceil': 'ceilf', 'floor': 'floorf', 'abs': 'fabsf'}
_UNARY_F64 = {'acos': 'acos', 'asin': 'asin', 'atan': 'atan', 'cos': 'cos', 'cosh': 'cosh', 'sin': 'sin',
              'sinh': 'sinh', 'tan': 'tan', 'tanh': 'tanh', 'exp': 'exp', 'log': 'log', 'log10': 'log10',
              'sqrt': 'sqrt', 'ceil': 'ceil', 'floor': 'floor', 'abs': 'fabs'}
_ABS_INT = {'int8': 'abs_8', 'int16': 'abs_16', 'int32': 'abs', 'int64': 'labs'}
# opveclib/expression.py:1657-1669
_INFIX = {'add': '+', 'sub': '-', 'mul': '*', 'div': '/', 'mod': '%', 'eq': '==', 'ne': '!=', 'lt': '<',
          'le': '<=', 'gt': '>', 'ge': '>=', 'and': '&&', 'or': '||'}
# opveclib/expression.py:1568-1572
_LIMITS = {('min_value', 'float32'): 'FLT_MIN', ('min_value', 'float64'): 'DBL_MIN',
           ('max_value', 'float32'): 'FLT_MAX', ('max_value', 'float64'): 'DBL_MAX',
           ('epsilon', 'float32'): 'FLT_EPSILON', ('epsilon', 'float64'): 'DBL_EPSILON'}


def ctype(dtype):
    # opveclib/expression.py:50-61 with int64_tf = long long (opveclib/dynamiclibop.h:18)
    return dtype.as_cstr()


def literal(value):
    """Python ``str()`` of the constant, as the reference names constants (opveclib/expression.py:328-329)."""
    if isinstance(value, float):
        if math.isinf(value):
            return 'INFINITY' if value > 0 else '(-INFINITY)'
        if math.isnan(value):
            return 'NAN'
        return repr(value)
    return str(int(value))


class _Emitter(object):
    def __init__(self, kernel):
        self.kernel = kernel
        self.names = {}
        self.lines = []
        self.depth = 2
        self.counter = 0

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
            # opveclib/expression.py:1293-1306
            self.names[id(node)] = 'position'
            shape = node.workgroup_shape
            blocks = [1]
            for d in range(len(shape) - 1, 0, -1):
                blocks.append(blocks[-1] * shape[d])
            blocks.reverse()
            vals, rem = [], 'worker_index'
            for b in blocks:
                vals.append('(' + rem + ')/' + str(b))
                rem = rem + ' % ' + str(b)
            self.put('const uint32_t position[' + str(len(shape)) + '] = {' + ', '.join(vals) + '};')
        elif k == 'variable' or k == 'cast':
            # opveclib/expression.py:1351-1352, 1386-1387
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + ' = ' + self.name(node.args[0]) + ';')
        elif k == 'local':
            # opveclib/expression.py:1794-1795
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + '[' + str(node.size) + '] = ' + self.name(node.args[0]) + ';')
        elif k == 'assign_var':
            # opveclib/expression.py:1422-1423
            self.put(self.name(node.args[0]) + ' = ' + self.name(node.args[1]) + ';')
        elif k == 'assign_tensor':
            # opveclib/expression.py:1881-1882
            self.put(self.name(node.args[0]) + '[' + self.name(node.args[1]) + '] = ' + self.name(node.args[2]) +
                     ';')
        elif k == 'read':
            # opveclib/expression.py:1904-1905
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + ' = ' + self.name(node.args[0]) + '[' +
                     self.name(node.args[1]) + '];')
        elif k == 'limit':
            self.names[id(node)] = _LIMITS[(node.attr['which'], node.dtype.name)]
        elif k == 'unary':
            # opveclib/expression.py:1479-1481
            fn, t = node.attr['fn'], node.dtype.name
            if fn == 'negate':
                f = '-'
            elif fn == 'not':
                f = '!'
            elif fn in ('isinf', 'isfinite', 'isnan'):
                f = 'std::' + fn
            elif fn == 'abs' and t in _ABS_INT:
                f = _ABS_INT[t]
            else:
                f = (_UNARY_F32 if t == 'float32' else _UNARY_F64)[fn]
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + ' = ' + f + '(' + self.name(node.args[0]) + ');')
        elif k == 'binary':
            # opveclib/expression.py:1739-1742 with the forms of 1648-1672
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
            else:
                rhs = '(' + x + ' ' + _INFIX[fn] + ' ' + y + ')'
            n = self.fresh(node)
            self.put(ctype(node.dtype) + ' ' + n + ' = ' + rhs + ';')
        elif k == 'for':
            # opveclib/expression.py:1996-2006
            i, a, b, s = [self.name(x) for x in node.args]
            self.put('for(' + i + ' = ' + a + '; ((' + i + ' < ' + b + ')&&(' + s + '>0)) || ((' + i + ' > ' + b +
                     ')&&(' + s + '<0)); ' + i + '+=' + s + '){')
            self.depth += 1
            self.block(node.body)
            self.depth -= 1
            self.put('}')
        elif k == 'if':
            # opveclib/expression.py:2064-2065, 2115-2116, 2160-2161, 2182-2183
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


def emit_cpp(kernel, function_name):
    """C++ source with ``extern "C" void <function_name>(const void* const* ins, void* const* outs, uint32_t
    num_threads, uint32_t thread_index)``: thread ``thread_index`` of ``num_threads`` processes its contiguous
    block of workers, block = ceil(W / num_threads) (opveclib/expression.py:582-590, 667-669)."""
    em = _Emitter(kernel)
    em.block(kernel.body)
    params, casts = [], []
    for n in kernel.inputs:
        i = n.attr['io_index']
        params.append('const ' + ctype(n.dtype) + '* in' + str(i))
        casts.append('(const ' + ctype(n.dtype) + '*)ins[' + str(i) + ']')
    for n in kernel.outputs:
        i = n.attr['io_index']
        params.append(ctype(n.dtype) + '* out' + str(i))
        casts.append('(' + ctype(n.dtype) + '*)outs[' + str(i) + ']')
    w = kernel.num_workers
    src = [
        '// generated by the oracle',
        '#include <stdint.h>', '#include <stdlib.h>', '#include <math.h>', '#include <cmath>', '#include <cfloat>',
        '#define abs_8(x) abs(x)', '#define abs_16(x) abs(x)',
        'static void body_' + function_name + '(' + ', '.join(params) + ', uint32_t block_size, uint32_t '
        'thread_index){',
        '    uint32_t start = thread_index * block_size;',
        '    uint32_t end = start + block_size;',
        '    if (end > ' + str(w) + 'u || end < start) end = ' + str(w) + 'u;',
        '    for(uint32_t worker_index=start; worker_index < end; worker_index++){',
    ] + em.lines + [
        '    }',
        '}',
        'extern "C" void ' + function_name + '(const void* const* ins, void* const* outs, uint32_t num_threads, '
        'uint32_t thread_index){',
        '    uint32_t block_size = ' + str(w) + 'u / num_threads;',
        '    if(' + str(w) + 'u % num_threads > 0) block_size += 1;',
        '    body_' + function_name + '(' + ', '.join(casts) + ', block_size, thread_index);',
        '}', '']
    return '\n'.join(src)
