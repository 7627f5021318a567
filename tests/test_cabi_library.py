"""The C-ABI launcher library loads without a GPU and exports every entry point its header declares."""
import ctypes
import os
import re

from opveclib_b200 import compiler, launcher

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'ovl_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(ovl_[a-z0-9_]+)\s*\(', text)))


def test_library_builds_and_exports_all_declared_symbols():
    path = compiler.build_launcher()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), name + ' is declared in include/ovl_b200.h but not exported'
    assert sorted(launcher.EXPORTS) == sorted(n for n in declared if n in launcher.EXPORTS)
    missing_in_binding = [n for n in declared if n not in launcher.EXPORTS]
    assert missing_in_binding == [] or all(n.endswith('_static') for n in missing_in_binding), missing_in_binding


def test_status_strings_and_size_queries_work_without_a_device():
    lib = launcher.library()
    assert b'sm_100a' in lib.ovl_version()
    assert lib.ovl_status_string(0) == b'ok'
    assert b'element count' in lib.ovl_status_string(2)
    assert b'wait expired' in lib.ovl_status_string(8)
    # 16-byte header + one 32-byte slot per tile: a line of up to 8192 elements is one tile, longer lines are
    # sized for tiles of 4096 (the finer of the two tilings in use)
    assert lib.ovl_scan_f32_scratch_bytes(1, 8192) == 16 + 32
    assert lib.ovl_scan_f32_scratch_bytes(3, 8193) == 16 + 32 * 9
    assert lib.ovl_scan_f32_scratch_bytes(4096, 8192) == 16 + 32 * 4096
    assert lib.ovl_scan_f32_scratch_bytes(1, 1 << 31) == 16 + 32 * (1 << 19)


def test_argument_validation_happens_before_any_cuda_call():
    lib = launcher.library()
    # null pointers and malformed arguments are rejected on the host
    assert lib.ovl_scan_f32(0, None, None, 1, 16, None, None, 0, None) == 4
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    assert lib.ovl_scan_f32(7, p, p, 1, 16, None, None, 0, None) == 11      # unknown op
    assert lib.ovl_scan_f32(0, p, p, 2, 16, p, None, 0, None) == 11         # carry needs a single line
    assert lib.ovl_scan_f32(0, p, p, 1, 16, None, None, 0, None) == 7       # scratch missing
    assert lib.ovl_reduce_f32(0, p, 0, p, p, 1 << 20, None) == 11           # empty reduction
    assert lib.ovl_launch(None, None, 0, None, 0, None, 0, None) == 4
    assert lib.ovl_kernel_create(None, None, None) == 4


def test_kernel_cache_is_keyed_by_structure():
    import numpy as np
    import cases
    ns = cases.impl()
    a = compiler.kernel_name(cases.c1_chain(ns, np.zeros(64, np.float32)).kernel)
    b = compiler.kernel_name(cases.c1_chain(ns, np.ones(64, np.float32)).kernel)
    c = compiler.kernel_name(cases.c1_chain(ns, np.zeros(128, np.float32)).kernel)
    assert a == b and a != c and a.startswith('f')
