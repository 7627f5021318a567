"""ctypes binding of the C-ABI launcher library (include/ovl_b200.h)."""
import ctypes
import os

from . import compiler


class OvlTensor(ctypes.Structure):
    _fields_ = [('data', ctypes.c_void_p), ('dtype', ctypes.c_int32), ('len', ctypes.c_uint64)]


class OvlKernelSpec(ctypes.Structure):
    _fields_ = [('symbol', ctypes.c_char_p), ('grid_x', ctypes.c_uint32), ('block_x', ctypes.c_uint32),
                ('dynamic_smem_bytes', ctypes.c_uint32), ('n_inputs', ctypes.c_uint32),
                ('n_outputs', ctypes.c_uint32), ('dtypes', ctypes.POINTER(ctypes.c_int32)),
                ('lens', ctypes.POINTER(ctypes.c_uint64)), ('align_bytes', ctypes.POINTER(ctypes.c_uint32)),
                ('scratch_bytes', ctypes.c_uint64), ('scratch_zero_bytes', ctypes.c_uint64),
                ('flags', ctypes.c_uint32)]


KERNEL_COOPERATIVE = 1
PEER_HANDLE_BYTES = 64
MAX_PEERS = 8


class OvlPeerExchange(ctypes.Structure):
    _fields_ = [('buffers', ctypes.c_void_p * MAX_PEERS), ('world', ctypes.c_uint32), ('rank', ctypes.c_uint32),
                ('epoch', ctypes.c_uint32)]


EXPORTS = ['ovl_version', 'ovl_status_string', 'ovl_last_cuda_error', 'ovl_device_sm_count', 'ovl_module_load',
           'ovl_module_load_file', 'ovl_module_unload', 'ovl_kernel_create', 'ovl_kernel_destroy', 'ovl_launch',
           'ovl_profile', 'ovl_run_host', 'ovl_read_kernel_status', 'ovl_scan_f32_scratch_bytes', 'ovl_scan_f32',
           'ovl_reduce_f32_scratch_bytes', 'ovl_reduce_f32', 'ovl_scan_f32_static', 'ovl_scan_f32_static_status', 'ovl_scan_f32_begin',
           'ovl_scan_f32_finish', 'ovl_selftest_scan_timeout', 'ovl_peer_buffer_bytes', 'ovl_peer_alloc',
           'ovl_peer_open', 'ovl_peer_close', 'ovl_peer_free', 'ovl_scan_f32_begin_peer', 'ovl_scan_f32_finish_peer']

_lib = None


class OvlError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        lib = library()
        msg = lib.ovl_status_string(status).decode()
        if status == 5:
            msg += ' %d' % lib.ovl_last_cuda_error()
        super(OvlError, self).__init__(what + ': ' + msg + ' (status %d)' % status)


def library():
    """Load libovl_b200.so (building it first if the source is newer and nvcc is present).  There is no
    fallback: without the library nothing can run."""
    global _lib
    if _lib is not None:
        return _lib
    path = compiler.LIB_PATH
    if os.path.exists(compiler.nvcc_path):
        # (returns at once when the library is newer than its sources)
        path = compiler.build_launcher(force=bool(os.environ.get('OVL_B200_REBUILD')))
    elif not os.path.exists(path):
        raise RuntimeError('libovl_b200.so is missing and there is no nvcc to build it: ' + path)
    lib = ctypes.CDLL(path)
    vp, u64, u32, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32
    tp = ctypes.POINTER(OvlTensor)
    lib.ovl_version.restype = ctypes.c_char_p
    lib.ovl_status_string.restype = ctypes.c_char_p
    lib.ovl_status_string.argtypes = [ctypes.c_int]
    lib.ovl_last_cuda_error.restype = ctypes.c_int
    lib.ovl_device_sm_count.argtypes = [ctypes.POINTER(ctypes.c_int)]
    lib.ovl_module_load.argtypes = [vp, ctypes.c_size_t, ctypes.POINTER(vp)]
    lib.ovl_module_load_file.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.ovl_module_unload.argtypes = [vp]
    lib.ovl_kernel_create.argtypes = [vp, ctypes.POINTER(OvlKernelSpec), ctypes.POINTER(vp)]
    lib.ovl_kernel_destroy.argtypes = [vp]
    lib.ovl_launch.argtypes = [vp, tp, ctypes.c_size_t, tp, ctypes.c_size_t, vp, u64, vp]
    lib.ovl_profile.argtypes = [vp, tp, ctypes.c_size_t, tp, ctypes.c_size_t, vp, u64, vp, u32,
                                ctypes.POINTER(ctypes.c_float)]
    lib.ovl_run_host.argtypes = [vp, tp, ctypes.c_size_t, tp, ctypes.c_size_t, u32, ctypes.POINTER(ctypes.c_float)]
    lib.ovl_read_kernel_status.argtypes = [vp, vp, ctypes.POINTER(i32)]
    lib.ovl_scan_f32_scratch_bytes.restype = u64
    lib.ovl_scan_f32_scratch_bytes.argtypes = [u64, u64]
    lib.ovl_scan_f32.argtypes = [ctypes.c_int, vp, vp, u64, u64, vp, vp, u64, vp]
    lib.ovl_reduce_f32_scratch_bytes.restype = u64
    lib.ovl_reduce_f32_scratch_bytes.argtypes = [u64]
    lib.ovl_reduce_f32.argtypes = [ctypes.c_int, vp, u64, vp, vp, u64, vp]
    lib.ovl_scan_f32_begin.argtypes = [ctypes.c_int, vp, u64, vp, vp, u64, vp]
    lib.ovl_scan_f32_finish.argtypes = [ctypes.c_int, vp, vp, u64, vp, vp, u64, vp]
    lib.ovl_selftest_scan_timeout.argtypes = [vp, vp, u64, vp, u64, vp]
    pxp = ctypes.POINTER(OvlPeerExchange)
    lib.ovl_peer_buffer_bytes.restype = u64
    lib.ovl_peer_alloc.argtypes = [ctypes.POINTER(vp), ctypes.c_char_p]
    lib.ovl_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.ovl_peer_close.argtypes = [vp]
    lib.ovl_peer_free.argtypes = [vp]
    lib.ovl_scan_f32_begin_peer.argtypes = [ctypes.c_int, vp, u64, vp, vp, u64, pxp, vp]
    lib.ovl_scan_f32_finish_peer.argtypes = [ctypes.c_int, vp, vp, u64, vp, u64, pxp, vp]
    lib.ovl_scan_f32_static.argtypes = [ctypes.c_int, vp, vp, u64, u64, vp, vp]
    lib.ovl_scan_f32_static_status.argtypes = [vp, ctypes.POINTER(i32)]
    _lib = lib
    return lib


def check(status, what):
    if status != 0:
        raise OvlError(status, what)


def tensor_array(items):
    """ctypes array of OvlTensor from (pointer, dtype code, element count) triples."""
    arr = (OvlTensor * max(1, len(items)))()
    for i, (ptr, code, n) in enumerate(items):
        arr[i].data = ptr
        arr[i].dtype = code
        arr[i].len = n
    return arr


class Module(object):
    """A cubin loaded into the current device's context."""

    def __init__(self, path):
        self.handle = ctypes.c_void_p()
        check(library().ovl_module_load_file(path.encode(), ctypes.byref(self.handle)), 'loading ' + path)


class Kernel(object):
    """One launchable kernel: symbol + signature + launch shape."""

    def __init__(self, module, symbol, grid, block, dtypes, lens, n_inputs, aligns=None, scratch_bytes=0,
                 scratch_zero_bytes=0, smem=0, cooperative=False):
        n = len(dtypes)
        self._dt = (ctypes.c_int32 * max(1, n))(*dtypes)
        self._ln = (ctypes.c_uint64 * max(1, n))(*lens)
        self._al = (ctypes.c_uint32 * max(1, n))(*(aligns or [0] * n))
        self._sym = symbol.encode()
        spec = OvlKernelSpec(self._sym, grid, block, smem, n_inputs, n - n_inputs, self._dt, self._ln, self._al,
                             scratch_bytes, scratch_zero_bytes, KERNEL_COOPERATIVE if cooperative else 0)
        self.handle = ctypes.c_void_p()
        self.module = module
        self.scratch_bytes = scratch_bytes
        self.symbol = symbol
        self.grid = grid
        self.n_inputs = n_inputs
        self.n_outputs = n - n_inputs
        check(library().ovl_kernel_create(module.handle, ctypes.byref(spec), ctypes.byref(self.handle)),
              'creating kernel ' + symbol)

    def launch(self, ins, n_in, outs, n_out, scratch_ptr, scratch_bytes, stream):
        """Enqueue one launch; returns the OvlStatus."""
        return library().ovl_launch(self.handle, ins, n_in, outs, n_out, scratch_ptr, scratch_bytes, stream)

    def profile(self, ins, n_in, outs, n_out, scratch_ptr, scratch_bytes, stream, iterations):
        ms = (ctypes.c_float * max(1, iterations))()
        st = library().ovl_profile(self.handle, ins, n_in, outs, n_out, scratch_ptr, scratch_bytes, stream,
                                   iterations, ms)
        return st, list(ms)[:iterations]
