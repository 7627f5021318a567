"""Local runtime environment: version, logger, toolchain paths and the compiled-kernel cache directory.

Same knobs as opveclib/local.py:18-63 (``CUDA_HOME``, ``OPVECLIB_HOME``, ``OPVECLIB_CXX``) with
``OVL_B200_HOME`` taking precedence for the cache location.  The default cache lives inside the package tree
so that pre-built cubins travel with a copy of the source tree.
"""
import logging
import os

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
