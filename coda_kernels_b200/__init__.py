"""B200-native kernels behind the fused-linear operators of ``coda.kernels.functional``.

Importing the package loads ``libcoda_b200.so`` (hand-written sm_100a kernels,
C ABI in ``include/coda_b200.h``); there is no CPU or eager fallback.
"""

from . import functional, ops, rope_utils
from ._lib import LIB_PATH, CodaB200Error, set_option
from .functional import (
    linear_cross_entropy,
    linear_cross_entropy_forward,
    linear_qknorm_rope,
    linear_sigmoid,
    linear_swiglu,
)
from .rope_utils import make_rope_frequencies

__all__ = [
    "functional",
    "ops",
    "rope_utils",
    "LIB_PATH",
    "CodaB200Error",
    "set_option",
    "linear_swiglu",
    "linear_sigmoid",
    "linear_cross_entropy",
    "linear_cross_entropy_forward",
    "linear_qknorm_rope",
    "make_rope_frequencies",
]
