"""Example operators written in the operator language (counterparts of opveclib/examples/__init__.py; the
triangle-counting example lives in :mod:`opveclib_b200.examples.graph`, as the reference keeps it out of the
package namespace too)."""
from .accumulate import accumulate, cumsum, cumprod
from .expm1 import expm1, expm1_grad
from .log1p import log1p, log1p_grad
from .lstm import lstm, lstm_grad
from .conv1d import conv_1d
