"""Same names as coda/kernels/functional/swiglu.py of the reference, implemented by coda_kernels_b200.functional.swiglu."""

from coda_kernels_b200.functional.swiglu import *  # noqa: F401,F403
from coda_kernels_b200.functional import swiglu as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
