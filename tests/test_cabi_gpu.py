"""The C-ABI entry points called directly (ctypes), as a non-Python host would: module load, kernel creation,
signature checks, device-pointer launch, timed launches, and the host-buffer run with the contract of the
reference harness (opveclib/testcudaop.cc:60-395: host pointers in, outputs pre-filled with 0xFE, host pointers
out)."""
import ctypes

import numpy as np
import pytest

import cases
from helpers import DRYRUN, assert_exact
from opveclib_b200 import compiler, launcher

pytestmark = pytest.mark.gpu

F32 = 2


def _shift_kernel(n):
    ns = cases.impl()
    op = cases.user_ops(ns).shift_cyclic(np.zeros(n, np.float32))
    cubin, meta = compiler.compile_kernel(op.kernel)
    return cubin, meta


def _host_tensors(arrays):
    return launcher.tensor_array([(a.ctypes.data, F32, a.size) for a in arrays])


def test_kernel_is_compiled_with_metadata():
    cubin, meta = _shift_kernel(5000)
    assert cubin.endswith('.cubin') and meta['gen']['symbol'].endswith('_gen') and meta['gen']['items'] == 5000
    assert meta['vec'] is not None and meta['vec']['lanes'] == 4          # aligned vector loads of the input


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_run_host_profile_and_signature_errors():
    import torch
    torch.cuda.init()
    lib = launcher.library()
    n = 5000
    cubin, meta = _shift_kernel(n)
    module = launcher.Module(cubin)
    kernel = launcher.Kernel(module, meta['gen']['symbol'], 8, 256, [F32, F32], [n, n], 1)

    # host buffers in and out
    x = np.random.RandomState(0).uniform(-1, 1, n).astype(np.float32)
    y = np.zeros(n, np.float32)
    ms = (ctypes.c_float * 3)()
    st = lib.ovl_run_host(kernel.handle, _host_tensors([x]), 1, _host_tensors([y]), 1, 3, ms)
    assert st == 0, lib.ovl_status_string(st)
    assert_exact(y, np.roll(x, 1), 'ovl_run_host shift_cyclic')
    assert all(0 < t < 100 for t in ms)

    # signature checks: arity, element count, dtype, null data
    assert lib.ovl_run_host(kernel.handle, _host_tensors([x, x]), 2, _host_tensors([y]), 1, 1, None) == 1
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.empty_like(d_x)
    stream = torch.cuda.current_stream().cuda_stream
    good_in = launcher.tensor_array([(d_x.data_ptr(), F32, n)])
    good_out = launcher.tensor_array([(d_y.data_ptr(), F32, n)])
    assert lib.ovl_launch(kernel.handle, good_in, 1, good_out, 0, None, 0, stream) == 1                 # arity
    assert lib.ovl_launch(kernel.handle, launcher.tensor_array([(d_x.data_ptr(), F32, n - 1)]), 1, good_out, 1, None, 0,
                          stream) == 2                                                                    # length
    assert lib.ovl_launch(kernel.handle, launcher.tensor_array([(d_x.data_ptr(), 3, n)]), 1, good_out, 1, None, 0,
                          stream) == 3                                                                    # dtype
    assert lib.ovl_launch(kernel.handle, launcher.tensor_array([(None, F32, n)]), 1, good_out, 1, None, 0, stream) == 4

    # device pointers, asynchronous on the caller's stream
    assert lib.ovl_launch(kernel.handle, good_in, 1, good_out, 1, None, 0, stream) == 0
    torch.cuda.synchronize()
    assert_exact(d_y.cpu().numpy(), np.roll(x, 1), 'ovl_launch shift_cyclic')
    times = (ctypes.c_float * 4)()
    assert lib.ovl_profile(kernel.handle, good_in, 1, good_out, 1, None, 0, stream, 4, times) == 0
    assert all(0 < t < 100 for t in times)

    # the vectorised variant refuses a misaligned pointer instead of faulting
    vec = launcher.Kernel(module, meta['vec']['symbol'], 8, 256, [F32, F32], [n, n], 1, [16, 0])
    big = torch.zeros(n + 1, dtype=torch.float32, device='cuda')
    off_in = launcher.tensor_array([(big.data_ptr() + 4, F32, n)])
    assert lib.ovl_launch(vec.handle, off_in, 1, good_out, 1, None, 0, stream) == 9
    assert lib.ovl_launch(vec.handle, good_in, 1, good_out, 1, None, 0, stream) == 0
    torch.cuda.synchronize()
    assert_exact(d_y.cpu().numpy(), np.roll(x, 1), 'vectorised shift_cyclic')

    # unknown symbol, sm count, unload
    spec_fail = pytest.raises(launcher.OvlError)
    with spec_fail:
        launcher.Kernel(module, 'no_such_kernel', 1, 32, [F32], [1], 1)
    sms = ctypes.c_int(0)
    assert lib.ovl_device_sm_count(ctypes.byref(sms)) == 0 and sms.value > 0
    assert lib.ovl_kernel_destroy(kernel.handle) == 0


@pytest.mark.skipif(DRYRUN, reason='needs a device')
def test_evaluate_falls_back_to_the_scalar_kernel_for_misaligned_tensors():
    """A torch view that starts 4 bytes into an allocation cannot use 128-bit accesses; the runtime picks the
    generic variant and the result is the same."""
    import torch
    ns = cases.impl()
    base = torch.arange(0, 4097, dtype=torch.float32, device='cuda')
    view = base[1:]
    assert view.data_ptr() % 16 != 0
    out = ns.ovl.evaluate(cases.c1_chain(ns, view))
    ref = ns.ovl.evaluate(cases.c1_chain(ns, view.clone()))
    assert torch.equal(out, ref)
