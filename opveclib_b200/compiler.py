"""nvcc driver and the on-disk kernel cache.

Kernels are cached as ``<cache>/f<sha224>.cubin`` plus ``f<sha224>.json`` (launch metadata), keyed by the
canonical text of the kernel IR, the library version and the template version - the counterpart of the
reference's ``~/.opveclib/<version>/f<sha224>_generic_cuda.so`` cache (opveclib/operator.py:357-358,
2065-2096).  The reference compiles with ``nvcc -O3 --use_fast_math`` and no ``-arch``; here the only target is
sm_100a, FMA contraction is off and fast-math is never used, so that fp32 results match the reference's C++
operator.
"""
import hashlib
import json
import os
import subprocess
import threading

from . import cuda_emit
from .local import cache_directory, nvcc_path, gpu_arch_flags, version, logger

_PKG = os.path.dirname(os.path.abspath(__file__))
TEMPLATE_DIR = os.path.join(_PKG, 'csrc', 'templates')
LIB_DIR = os.path.join(_PKG, 'lib')
LIB_PATH = os.path.join(LIB_DIR, 'libovl_b200.so')
LAUNCHER_SRC = os.path.join(_PKG, 'csrc', 'ovl_launcher.cu')
NVCC_FLAGS = ['-O3', '--fmad=false', '-std=c++17', '-lineinfo', '-diag-suppress', '177,186,550']
_lock = threading.Lock()


def _template_stamp():
    """Digest of everything that shapes generated code: the device templates and the emitters themselves."""
    h = hashlib.sha224()
    paths = [os.path.join(TEMPLATE_DIR, fn) for fn in sorted(os.listdir(TEMPLATE_DIR))]
    paths += [os.path.join(_PKG, fn) for fn in ('cuda_emit.py', 'cuda_pack.py', 'patterns.py', 'access.py')]
    for path in paths:
        with open(path, 'rb') as f:
            h.update(f.read())
    return h.hexdigest()[:16]


_STAMP = None


#: environment variables read while a kernel's source is generated
EMIT_SWITCHES = ('OVL_RED_SPLIT', 'OVL_RED_LAYOUT')


def kernel_name(kernel, math='exact'):
    """'f' + sha224 of (kernel text, version, templates, math lowering) - stable across processes."""
    global _STAMP
    if _STAMP is None:
        _STAMP = _template_stamp()
    key = kernel.text() + '|' + version + '|' + cuda_emit.TEMPLATE_VERSION + '|' + _STAMP
    if math != 'exact':
        key += '|math=' + math
    # switches that change the generated source name a different kernel (unset: the usual name)
    for switch in EMIT_SWITCHES:
        if os.environ.get(switch):
            key += '|' + switch + '=' + os.environ[switch]
    return 'f' + hashlib.sha224(key.encode('utf-8')).hexdigest()[:48]


def _run(cmd):
    try:
        return subprocess.check_output(cmd, stderr=subprocess.STDOUT, universal_newlines=True)
    except subprocess.CalledProcessError as exc:
        logger.error('nvcc error: ' + exc.output)
        raise RuntimeError('nvcc failed:\n' + exc.output)


def compile_kernel(kernel, math='exact'):
    """Generate and compile one kernel (or fetch it from the cache).  Returns (cubin path, metadata)."""
    name = kernel_name(kernel, math)
    cubin = os.path.join(cache_directory, name + '.cubin')
    meta_path = os.path.join(cache_directory, name + '.json')
    if os.path.exists(cubin) and os.path.exists(meta_path):
        with open(meta_path) as f:
            return cubin, json.load(f)
    logger.debug('Compiling CUDA for kernel ' + kernel.name + ' as ' + name)
    source, meta = cuda_emit.emit_cuda(kernel, name, math)
    meta['name'] = name
    meta['kernel'] = kernel.name
    meta['math'] = math
    src_path = os.path.join(cache_directory, name + '.cu')
    with open(src_path, 'w') as f:
        f.write(source)
    tmp = cubin + '.%d.%d.tmp' % (os.getpid(), threading.get_ident())
    _run([nvcc_path] + gpu_arch_flags + NVCC_FLAGS + ['-cubin', '-I' + TEMPLATE_DIR, '-o', tmp, src_path])
    os.replace(tmp, cubin)
    tmpm = meta_path + '.%d.%d.tmp' % (os.getpid(), threading.get_ident())
    with open(tmpm, 'w') as f:
        json.dump(meta, f)
    os.replace(tmpm, meta_path)
    return cubin, meta


def _launcher_stamp(deps):
    h = hashlib.sha224()
    for d in sorted(deps):
        if os.path.exists(d):
            with open(d, 'rb') as f:
                h.update(f.read())
    h.update(' '.join(gpu_arch_flags + NVCC_FLAGS).encode('utf-8'))
    return h.hexdigest()


def build_launcher(force=False):
    """Compile csrc/ovl_launcher.cu into lib/libovl_b200.so for sm_100a (no GPU needed).  The library is rebuilt
    when the content of its sources differs from what it was built from (a digest kept beside it - file times do
    not survive a copy of the tree)."""
    with _lock:
        os.makedirs(LIB_DIR, exist_ok=True)
        deps = [LAUNCHER_SRC, os.path.join(_PKG, '..', 'include', 'ovl_b200.h')] + \
            [os.path.join(TEMPLATE_DIR, fn) for fn in os.listdir(TEMPLATE_DIR)]
        stamp = _launcher_stamp(deps)
        stamp_path = LIB_PATH + '.stamp'
        if not force and os.path.exists(LIB_PATH) and os.path.exists(stamp_path):
            with open(stamp_path) as f:
                if f.read().strip() == stamp:
                    return LIB_PATH
        tmp = LIB_PATH + '.%d.tmp' % os.getpid()
        _run([nvcc_path] + gpu_arch_flags + NVCC_FLAGS + ['-shared', '-Xcompiler', '-fPIC', '-o', tmp, LAUNCHER_SRC])
        os.replace(tmp, LIB_PATH)
        with open(stamp_path + '.%d.tmp' % os.getpid(), 'w') as f:
            f.write(stamp)
        os.replace(stamp_path + '.%d.tmp' % os.getpid(), stamp_path)
        return LIB_PATH
