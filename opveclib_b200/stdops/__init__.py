"""Standard operators written in the operator language (counterpart of opveclib/stdops)."""
from .math import (neg, tanh, sin, cos, tan, sigmoid, split, concat, add, sub, mul, div, mod, equal, not_equal, less,
                   less_equal, greater, greater_equal)
