"""TEST INFRASTRUCTURE - CPU oracle, never part of the product path.

Compiles the C++ emitted by :mod:`oracle.cpp_emit` with g++ and runs it on host threads through
``oracle/harness.cc``, one operator after the other exactly like the reference's ``profile`` loop over the
operator graph with ``target_language='cpp'`` and no merging (opveclib/operator.py:2256-2335): leaf inputs are
numpy arrays, every operator output is a fresh numpy buffer pre-filled with 0xFE bytes
(opveclib/testcop.cc:105-113), later operators read the buffers of earlier ones.

Build flags: ``-O2 -ffp-contract=off`` by default - no floating point contraction, so results are those of the
reference's own unoptimised build (opveclib/operator.py:2051-2055), which ``flags='reference'`` reproduces.
"""
import ctypes
import hashlib
import os
import subprocess

import numpy as np

from opveclib_b200.opgraph import build_op_dag
from . import cpp_emit

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, '_build')
FLAG_SETS = {
    'fast': ['-O2', '-ffp-contract=off'],
    'native': ['-O3', '-march=native', '-ffp-contract=off'],
    'reference': ['-g'],
}
_harness = None
_libs = {}


def _cxx():
    return os.getenv('OPVECLIB_CXX', 'g++')


def harness():
    """Build (once) and load the thread harness."""
    global _harness
    if _harness is None:
        os.makedirs(_BUILD, exist_ok=True)
        so = os.path.join(_BUILD, 'liboracle_harness.so')
        src = os.path.join(_HERE, 'harness.cc')
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            tmp = so + '.%d.tmp' % os.getpid()
            subprocess.check_output([_cxx(), '-O2', '-fPIC', '-shared', '-std=c++11', '-pthread', '-o', tmp, src,
                                     '-ldl'], stderr=subprocess.STDOUT)
            os.replace(tmp, so)
        lib = ctypes.CDLL(so)
        lib.ovl_oracle_run.restype = ctypes.c_int
        lib.ovl_oracle_run.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p),
                                       ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint32,
                                       ctypes.POINTER(ctypes.c_double), ctypes.c_uint32]
        lib.ovl_oracle_hardware_threads.restype = ctypes.c_uint32
        _harness = lib
    return _harness


def hardware_threads():
    return int(harness().ovl_oracle_hardware_threads())


def compile_kernel(kernel, flags='fast'):
    """g++ the oracle source of one kernel; returns (library path, entry point name)."""
    digest = hashlib.sha224((kernel.text() + '|' + flags).encode('utf-8')).hexdigest()[:40]
    fname = 'o' + digest
    key = (fname, flags)
    if key in _libs:
        return _libs[key]
    os.makedirs(_BUILD, exist_ok=True)
    so = os.path.join(_BUILD, fname + '.so')
    if not os.path.exists(so):
        src_path = os.path.join(_BUILD, fname + '.cpp')
        with open(src_path, 'w') as f:
            f.write(cpp_emit.emit_cpp(kernel, fname))
        tmp = so + '.%d.tmp' % os.getpid()
        try:
            subprocess.check_output([_cxx(), '-fPIC', '-std=c++11', '-shared'] + FLAG_SETS[flags] +
                                    ['-o', tmp, src_path], stderr=subprocess.STDOUT, universal_newlines=True)
        except subprocess.CalledProcessError as exc:
            raise RuntimeError('oracle c++ compiler error:\n' + exc.output)
        os.replace(tmp, so)
    _libs[key] = (so, fname)
    return _libs[key]


def run_kernel(kernel, inputs, num_threads=0, iterations=1, flags='fast'):
    """Run one kernel on numpy inputs.  Returns (list of output arrays, per-iteration milliseconds)."""
    so, fname = compile_kernel(kernel, flags)
    ins = []
    for arr, t in zip(inputs, kernel.input_types):
        a = np.ascontiguousarray(arr, dtype=t.dtype.as_numpy())
        if a.size != t.size:
            raise ValueError('input has %d elements, operator expects %d' % (a.size, t.size))
        ins.append(a)
    if len(ins) != len(kernel.input_types):
        raise ValueError('wrong number of inputs')
    outs = []
    for t in kernel.output_types:
        buf = np.empty(t.shape, dtype=t.dtype.as_numpy())
        buf.view(np.uint8).fill(0xFE)
        outs.append(buf)
    in_ptrs = (ctypes.c_void_p * max(1, len(ins)))(*[a.ctypes.data for a in ins])
    out_ptrs = (ctypes.c_void_p * max(1, len(outs)))(*[a.ctypes.data for a in outs])
    ms = (ctypes.c_double * iterations)()
    rc = harness().ovl_oracle_run(so.encode(), fname.encode(), in_ptrs, out_ptrs, num_threads, ms, iterations)
    if rc != 0:
        raise RuntimeError('oracle harness failed with code %d' % rc)
    return outs, np.array(list(ms))


def profile(output_list, num_threads=0, iterations=1, flags='fast'):
    """Evaluate operator outputs on the CPU, unmerged.  Returns (arrays, {op position: ms per iteration})."""
    if not isinstance(output_list, (list, tuple)):
        output_list = [output_list]
    return run_dag(build_op_dag(*output_list), num_threads, iterations, flags)


def run_dag(dag, num_threads=0, iterations=1, flags='fast'):
    """Run an operator graph (merged or not) operator by operator."""
    buffers, times = [], {}
    for op_index, kernel in enumerate(dag.kernels):
        cur_inputs = []
        for ref in dag.references[op_index]:
            if ref.is_leaf:
                cur_inputs.append(np.asarray(dag.inputs[ref.dag_input_index]))
            else:
                cur_inputs.append(buffers[ref.op_index][ref.op_output_index])
        outs, ms = run_kernel(kernel, cur_inputs, num_threads, iterations, flags)
        buffers.append(outs)
        times[(op_index, kernel.name)] = ms
    return [buffers[o][k] for o, k in dag.outputs], times


def evaluate(output_list, num_threads=0, flags='fast'):
    """numpy result(s) of operator outputs computed by the CPU oracle; a single output comes back bare."""
    outs, _ = profile(output_list, num_threads, 1, flags)
    return outs[0] if len(outs) == 1 else outs
