"""Local runtime environment: version, logger, toolchain paths and the compiled-kernel cache directory.

Same knobs as opveclib/local.py:18-63 (``CUDA_HOME``, ``OPVECLIB_HOME``, ``OPVECLIB_CXX``) with
``OVL_B200_HOME`` taking precedence for the cache location.  The default cache lives inside the package tree
so that pre-built cubins travel with a copy of the source tree.
"""
import logging
import os
import threading

#: Version string; part of every kernel cache key
version = '0.1.0-b200'

#: The logger
logger = logging.getLogger('opveclib_b200')

cuda_directory = os.getenv('CUDA_HOME', '/usr/local/cuda')
nvcc_path = os.path.join(cuda_directory, 'bin', 'nvcc')

_package_dir = os.path.dirname(os.path.abspath(__file__))
_base_cache_directory = os.getenv('OVL_B200_HOME', os.getenv('OPVECLIB_HOME', os.path.join(_package_dir, '_kcache')))

#: Directory where compiled kernels are cached
cache_directory = os.path.join(_base_cache_directory, version)
os.makedirs(cache_directory, exist_ok=True)

#: Host C++ compiler
cxx = os.getenv('OPVECLIB_CXX', 'g++')

#: sm_100a is the only target
gpu_arch_flags = ['-gencode', 'arch=compute_100a,code=sm_100a']


def clear_op_cache():
    """Delete all cached kernels (files whose name starts with 'f', as in the reference)."""
    for filename in os.listdir(cache_directory):
        if filename[0] == 'f':
            os.remove(os.path.join(cache_directory, filename))


def _detect_cuda():
    if not os.path.exists(nvcc_path):
        logger.info('nvcc not found - kernels cannot be compiled')
        return False
    return True


#: True when the CUDA toolchain needed to compile kernels is present
cuda_enabled = _detect_cuda()


# ---------------------------------------------------------------------------------------------------------
# math lowering of generated kernels: 'exact' (CUDA's libm and IEEE division: results within an ulp or two of the
# reference's C++ operator) or 'tolerance' (fp32 division, exp, log, log10, sqrt, tanh with bounded error - division
# and sqrt within 1.8e-7 relative, the functions within rtol 1e-5 - and packed two-element arithmetic; several times fewer instructions
# for chains of transcendentals).  The reference's own CUDA path is built with --use_fast_math
# (opveclib/operator.py:2081); 'tolerance' is this backend's counterpart with stated bounds.
MATH_MODES = ('exact', 'tolerance')
_default_math = os.getenv('OVL_B200_MATH', 'exact')
if _default_math not in MATH_MODES:
    raise ValueError('OVL_B200_MATH must be one of ' + ', '.join(MATH_MODES))
_math_override = threading.local()


def get_math_mode():
    """The math lowering that ``evaluate`` / ``profile`` / ``as_torch`` use when not told otherwise."""
    stack = getattr(_math_override, 'stack', None)
    return stack[-1] if stack else _default_math


def set_math_mode(mode):
    """Set the process-wide default math lowering ('exact' or 'tolerance')."""
    global _default_math
    if mode not in MATH_MODES:
        raise ValueError('math mode must be one of ' + ', '.join(MATH_MODES))
    _default_math = mode


class math_mode(object):
    """``with ovl.math_mode('tolerance'): ...`` - the lowering for calls made by this thread inside the block."""

    def __init__(self, mode):
        if mode is not None and mode not in MATH_MODES:
            raise ValueError('math mode must be one of ' + ', '.join(MATH_MODES))
        self.mode = mode

    def __enter__(self):
        if not hasattr(_math_override, 'stack'):
            _math_override.stack = []
        _math_override.stack.append(self.mode if self.mode is not None else get_math_mode())
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        _math_override.stack.pop()
