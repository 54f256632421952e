"""Same names as coda/kernels/functional/cross_entropy.py of the reference, implemented by coda_kernels_b200.functional.cross_entropy."""

from coda_kernels_b200.functional.cross_entropy import *  # noqa: F401,F403
from coda_kernels_b200.functional import cross_entropy as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
