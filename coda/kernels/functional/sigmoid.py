"""Same names as coda/kernels/functional/sigmoid.py of the reference, implemented by coda_kernels_b200.functional.sigmoid."""

from coda_kernels_b200.functional.sigmoid import *  # noqa: F401,F403
from coda_kernels_b200.functional import sigmoid as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
