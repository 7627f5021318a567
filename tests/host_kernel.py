"""TEST INFRASTRUCTURE: run a generated element-wise kernel (``_gen`` or ``_vec``) on the HOST.

The generated ``.cu`` text is compiled by g++ against the stand-in headers of tests/host_shim (same names as the
device templates), with the CUDA launch geometry emulated by loops over blocks and threads.  Only kernels without
shared memory and barriers can run this way (the generic and the vectorised kernel); that is what is needed to check
the code generator's bodies - hoisted vector accesses, packed pairs, masks, selects - against the CPU oracle on a
machine without a GPU.
"""
import ctypes
import hashlib
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_DRIVER = r'''
thread_local ovl_host_dim3 blockIdx, threadIdx, gridDim, blockDim;
extern "C" void ovl_host_run(void (*kernel)(void**), void** args, unsigned grid, unsigned block) {
    gridDim = {grid, 1, 1};
    blockDim = {block, 1, 1};
    for (unsigned b = 0; b < grid; ++b)
        for (unsigned t = 0; t < block; ++t) {
            blockIdx = {b, 0, 0};
            threadIdx = {t, 0, 0};
            kernel(args);
        }
}
'''


def run(source, symbol, params, grid, block, ins, outs):
    """Compile ``source`` for the host and run kernel ``symbol`` (C parameter list ``params``: const T* in0 ...,
    T* out0 ...) over ``grid`` blocks of ``block`` threads on the numpy arrays ``ins`` / ``outs``."""
    names = [p.split()[-1] for p in params]
    casts = ', '.join('(%s)a[%d]' % (' '.join(p.replace('__restrict__', '').split()[:-1]), i)
                      for i, p in enumerate(params))
    glue = '\nextern "C" void ovl_host_entry(void** a) { %s(%s); }\n' % (symbol, casts)
    text = source.replace('extern "C" __global__', 'extern "C"') + _DRIVER + glue
    key = hashlib.sha1(text.encode()).hexdigest()[:16]
    build = os.path.join(tempfile.gettempdir(), 'ovl_host_kernels')
    os.makedirs(build, exist_ok=True)
    so = os.path.join(build, key + '.so')
    if not os.path.exists(so):
        cpp = os.path.join(build, key + '.cpp')
        with open(cpp, 'w') as f:
            f.write(text)
        subprocess.check_output([os.getenv('OPVECLIB_CXX', 'g++'), '-std=c++17', '-O1', '-ffp-contract=off', '-fPIC',
                                 '-shared', '-w', '-I' + os.path.join(_HERE, 'host_shim'), '-o', so, cpp],
                                stderr=subprocess.STDOUT)
    lib = ctypes.CDLL(so)
    arrays = list(ins) + list(outs)
    assert len(arrays) == len(names)
    ptrs = (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    entry = ctypes.cast(lib.ovl_host_entry, ctypes.c_void_p)
    lib.ovl_host_run.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint, ctypes.c_uint]
    lib.ovl_host_run(entry, ptrs, grid, block)
    return outs


def run_vec(kernel, math='tolerance'):
    """Emit ``kernel`` (a KernelIR) with the given math lowering and return a function ins -> outs that runs its
    vectorised variant on the host, plus the emitter's metadata."""
    from opveclib_b200 import cuda_emit
    source, meta = cuda_emit.emit_cuda(kernel, 'fhost', math)
    assert meta['vec'] is not None, 'kernel has no vectorised variant'
    # keep the preamble and the _vec kernel only (other variants may use shared memory)
    start = source.index('extern "C" __global__ void __launch_bounds__(' + str(meta['vec']['block']) + ') fhost_vec(')
    end = source.index('\n}\n', start) + 3
    head = source[:source.index('extern "C" __global__')]
    text = head + source[start:end]
    params = cuda_emit._params(kernel)

    def call(ins):
        outs = []
        for t in kernel.output_types:       # (pre-filled like the oracle's harness: elements no worker writes keep 0xFE)
            buf = np.empty(t.shape, dtype=t.dtype.as_numpy())
            buf.view(np.uint8).fill(0xFE)
            outs.append(buf)
        block = meta['vec']['block']
        grid = max(1, min((meta['vec']['items'] + block - 1) // block, 7))     # a few blocks: the loop strides
        run(text, 'fhost_vec', params, grid, block, [np.ascontiguousarray(a) for a in ins], outs)
        return outs
    return call, meta
