"""``coda.kernels.functional``: same module and function names as the reference (README.md:45-49)."""

from coda_kernels_b200.functional import (
    linear_cross_entropy,
    linear_cross_entropy_forward,
    linear_qknorm_rope,
    linear_sigmoid,
    linear_swiglu,
)

__all__ = [
    "linear_swiglu",
    "linear_sigmoid",
    "linear_cross_entropy",
    "linear_cross_entropy_forward",
    "linear_qknorm_rope",
]
