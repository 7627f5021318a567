"""B200-native backend for the Operator Vectorization Library: the reference's operator API
(opveclib/__init__.py:11-48) over an sm_100a CUDA code generator and a C-ABI launcher."""
# data types
from .dtypes import DType, TensorType
from .dtypes import float32, float64, int8, int16, int32, int64, uint8, uint16, uint32, uint64
# expressions
from .expr import Scalar, Variable, InputTensor, OutputTensor, PositionTensor, LocalTensor
# tensor functions
from .expr import position_in, output, output_like, zeros, ones
# scalar functions
from .expr import variable, cast
from .expr import min_value, max_value, epsilon
from .expr import arccos, arcsin, arctan, cos, cosh, sin, sinh, tan, tanh
from .expr import exp, log, log10, sqrt, ceil, absolute, floor, logical_not, isinf, isfinite, isnan
from .expr import minimum, maximum, power, arctan2, logical_and, logical_or
# control flow
from .expr import arange, if_, elif_, else_
# operators
from .opgraph import operator, gradient
from .runtime import evaluate, profile
from .torch_bridge import as_torch, as_tensorflow
# local runtime environment
from .local import version, logger, cuda_enabled, cache_directory, clear_op_cache
from .local import math_mode, set_math_mode, get_math_mode
