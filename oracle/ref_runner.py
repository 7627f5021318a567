"""TEST INFRASTRUCTURE - never part of the product path.

Runs a workload of ``oracle/_ref/manifest.json`` (the reference's own generated C++ operators, built by
oracle/build_ref.py) on numpy arrays, through the stand-in harness with the reference harness's contract: one
task per thread index on ``num_threads`` host threads per operator, operators in graph order, outputs pre-filled
with 0xFE.  Needs neither the reference tree nor its Python dependencies.
"""
import ctypes
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, '_ref')
_NP = {2: np.float32, 3: np.float64, 4: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 8: np.uint8, 9: np.uint16,
       10: np.uint32, 11: np.uint64}


class _TensorParam(ctypes.Structure):
    _fields_ = [('data', ctypes.c_void_p), ('dtype', ctypes.c_int), ('len', ctypes.c_size_t)]


_state = {}


def available(workload=None):
    path = os.path.join(REF, 'manifest.json')
    if not os.path.exists(path) or not os.path.exists(os.path.join(REF, 'libref_harness.so')):
        return False
    if workload is None:
        return True
    return workload in manifest()


def manifest():
    if 'manifest' not in _state:
        with open(os.path.join(REF, 'manifest.json')) as f:
            _state['manifest'] = json.load(f)
    return _state['manifest']


def _harness():
    if 'lib' not in _state:
        lib = ctypes.CDLL(os.path.join(REF, 'libref_harness.so'))
        lib.testCOperatorThreads.restype = ctypes.c_int32
        lib.testCOperatorThreads.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(_TensorParam),
                                             ctypes.c_size_t, ctypes.POINTER(_TensorParam), ctypes.c_size_t,
                                             ctypes.POINTER(ctypes.c_double), ctypes.c_size_t, ctypes.c_uint32]
        lib.refHardwareThreads.restype = ctypes.c_uint32
        _state['lib'] = lib
    return _state['lib']


def hardware_threads():
    return int(_harness().refHardwareThreads())


def run(workload, inputs, num_threads=0, variant='opt', iterations=1):
    """Execute a workload.  Returns (list of output arrays, total milliseconds per iteration summed over the
    workload's operators)."""
    entry = manifest()[workload]
    lib = _harness()
    buffers = []
    total_ms = np.zeros(iterations)
    leaves = []
    for arr, (code, shape) in zip(inputs, entry['inputs']):
        a = np.ascontiguousarray(arr, dtype=_NP[code])
        if list(a.shape) != list(shape):
            raise ValueError('input shape %s, workload expects %s' % (a.shape, shape))
        leaves.append(a)
    for op in entry['ops']:
        ins = []
        for ref in op['inputs']:
            ins.append(leaves[ref[1]] if ref[0] == 'L' else buffers[ref[1]][ref[2]])
        outs = [np.empty(shape, dtype=_NP[code]) for code, shape in op['out_types']]
        in_params = (_TensorParam * max(1, len(ins)))()
        for i, (a, (code, shape)) in enumerate(zip(ins, op['in_types'])):
            in_params[i] = _TensorParam(a.ctypes.data, code, a.size)
        out_params = (_TensorParam * max(1, len(outs)))()
        for i, (a, (code, shape)) in enumerate(zip(outs, op['out_types'])):
            out_params[i] = _TensorParam(a.ctypes.data, code, a.size)
        ms = (ctypes.c_double * iterations)()
        so = os.path.join(REF, op['lib'] + '_' + variant + '.so')
        err = lib.testCOperatorThreads(so.encode(), op['fn'].encode(), in_params, len(ins), out_params, len(outs), ms,
                                       iterations, num_threads)
        if err != 0:
            raise RuntimeError('reference operator %s failed with code %d' % (op['name'], err))
        total_ms += np.array(list(ms))
        buffers.append(outs)
    return [buffers[o][k] for o, k in entry['outputs']], total_ms
