"""Public operator API: drop-in for ``coda.kernels.functional`` (README.md:45-49 of the reference)."""

from . import cross_entropy, qknorm_rope, sigmoid, sigmoid_glu, swiglu
from .cross_entropy import linear_cross_entropy, linear_cross_entropy_forward
from .qknorm_rope import linear_qknorm_rope
from .sigmoid import linear_sigmoid
from .sigmoid_glu import linear_sigmoid_glu
from .swiglu import linear_swiglu

__all__ = [
    "linear_swiglu",
    "linear_sigmoid",
    "linear_sigmoid_glu",
    "linear_cross_entropy",
    "linear_cross_entropy_forward",
    "linear_qknorm_rope",
    "swiglu",
    "sigmoid",
    "cross_entropy",
    "qknorm_rope",
]
