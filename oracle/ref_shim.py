"""TEST INFRASTRUCTURE - never part of the product path.

Makes the unmodified reference importable and runnable in the development container (Python 3.12, no
TensorFlow), for generating golden vectors and the reference-built CPU operators under ``oracle/_ref``.  Nothing
here is used on a machine where the reference tree is absent.  The reference tree is never edited; every
accommodation lives in this process only:

* ``opveclib/local.py:15`` imports tensorflow -> a stub module that only answers ``test.is_built_with_cuda()``
  (False) and ``sysconfig.get_include()``;
* ``opveclib/language_pb2.py`` is protoc-3.0 era generated code -> pure-python protobuf implementation;
* ``inspect.getargspec`` (opveclib/operator.py:394) no longer exists -> alias of ``getfullargspec``;
* the decorator's bytecode walker assumes 3-byte opcodes (opveclib/operator.py:588-641) and is only a lint ->
  the decorator is replaced by one that builds the reference's ``_OpGenerator`` directly;
* numpy 2 refuses to store a ctypes structure into a structured array element
  (``cur_input_params[i] = _TensorParam(...)``, opveclib/operator.py:2289, 2303) -> the module's ``np.empty`` is
  wrapped so that arrays of ``_TensorParam`` accept such an assignment field by field;
* ``opveclib/testcop.cc`` needs TensorFlow headers -> ``oracle/ref_harness.cc`` is built in its place into the
  reference's cache directory, where ``profile`` looks for it first (opveclib/operator.py:2165-2167).

Call :func:`load` in a dedicated process (the environment variables it sets must not leak into a process that
imports torch or the product).
"""
import inspect
import os
import subprocess
import sys
import types

_HERE = os.path.dirname(os.path.abspath(__file__))
# where the reference tree lies: OVL_REFERENCE_ROOT, else a directory `reference` beside this repository
REFERENCE_ROOT = os.environ.get('OVL_REFERENCE_ROOT',
                                os.path.join(os.path.dirname(os.path.dirname(_HERE)), 'reference'))
REF_VERSION = '1.0.3-dev0'   # opveclib/local.py:18


def available():
    return os.path.isdir(os.path.join(REFERENCE_ROOT, 'opveclib'))


def build_harness(out_path):
    """Compile the stand-in harness against the reference's dynamiclibop.h, from where the reference lies."""
    src = os.path.join(_HERE, 'ref_harness.cc')
    subprocess.check_output([os.getenv('OPVECLIB_CXX', 'g++'), '-fPIC', '-shared', '-std=c++11', '-O2', '-pthread',
                             '-I' + os.path.join(REFERENCE_ROOT, 'opveclib'), '-o', out_path, src, '-ldl'],
                            stderr=subprocess.STDOUT)
    return out_path


def load(cache_home):
    """Import the reference with its cache directory under ``cache_home``.  Returns a namespace with
    ``ovl`` (the package), ``opmod`` (the ``opveclib.operator`` module), ``stdops``, ``cumsum``, ``cumprod``,
    ``expm1``, ``log1p``, ``conv_1d``, ``lstm``, ``lstm_grad``."""
    if not available():
        raise RuntimeError('reference tree not found at ' + REFERENCE_ROOT)
    os.environ['PROTOCOL_BUFFERS_PYTHON_IMPLEMENTATION'] = 'python'
    os.environ['OPVECLIB_HOME'] = cache_home
    os.makedirs(os.path.join(cache_home, REF_VERSION), exist_ok=True)

    tf = types.ModuleType('tensorflow')
    tf.test = types.SimpleNamespace(is_built_with_cuda=lambda: False)
    tf.sysconfig = types.SimpleNamespace(get_include=lambda: '')
    sys.modules['tensorflow'] = tf
    if not hasattr(inspect, 'getargspec'):
        inspect.getargspec = lambda f: tuple(inspect.getfullargspec(f)[:4])
    if REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, REFERENCE_ROOT)

    import opveclib
    opmod = sys.modules['opveclib.operator']

    def operator(forbid_none_valued_constants=True, name=None):
        def wrapper(op_function):
            op = opmod._OpGenerator(op_function, forbid_none_valued_constants, None)
            op.__name__ = op_function.__name__
            op.__doc__ = op_function.__doc__
            return op
        return wrapper

    opmod.operator = operator
    opveclib.operator = operator

    import ctypes
    import numpy

    class _ParamArray(numpy.ndarray):
        def __setitem__(self, key, value):
            if isinstance(value, ctypes.Structure):
                value = (value.data or 0, value.dtype, value.len)
            numpy.ndarray.__setitem__(self, key, value)

    class _NumpyProxy(object):
        def __getattr__(self, item):
            return getattr(numpy, item)

        @staticmethod
        def empty(shape, dtype=float, **kwargs):
            if dtype is opmod._TensorParam:
                return numpy.empty(shape, dtype=numpy.dtype(dtype)).view(_ParamArray)
            return numpy.empty(shape, dtype=dtype, **kwargs)

    opmod.np = _NumpyProxy()

    harness = os.path.join(cache_home, REF_VERSION, 'libtestcop.so.' + REF_VERSION)
    if not os.path.exists(harness):
        build_harness(harness)

    import opveclib.stdops as stdops
    ns = types.SimpleNamespace(ovl=opveclib, opmod=opmod, stdops=stdops)

    # examples: the test modules define the operators and import unittest/tensorflow (stubbed) only
    from opveclib.examples.test_accumulate import cumsum, cumprod, accumulate
    from opveclib.examples.test_expm1 import expm1
    from opveclib.examples.test_log1p import log1p
    ns.cumsum, ns.cumprod, ns.accumulate, ns.expm1, ns.log1p = cumsum, cumprod, accumulate, expm1, log1p
    # examples/conv1D.py runs a TensorFlow comparison at import time; take the operator definition only (the text
    # up to the first helper that follows it)
    with open(os.path.join(REFERENCE_ROOT, 'opveclib', 'examples', 'conv1D.py')) as f:
        text = f.read()
    text = text[:text.index('\ndef reference(')]
    scope = {'__name__': 'ref_conv1d'}
    exec(compile(text, 'ref_conv1d.py', 'exec'), scope)
    ns.conv_1d = scope['conv_1d']

    # lstm/lstm.py uses python-2 integer division at lines 35 and 66; run its text with '//' instead
    with open(os.path.join(REFERENCE_ROOT, 'lstm', 'lstm.py')) as f:
        text = f.read().replace("concat.shape[1]/4", "concat.shape[1]//4")
    scope = {'__name__': 'ref_lstm'}
    exec(compile(text, 'ref_lstm.py', 'exec'), scope)
    ns.lstm, ns.lstm_grad = scope['lstm'], scope['lstm_grad']
    return ns
