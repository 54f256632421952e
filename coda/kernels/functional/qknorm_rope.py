"""Same names as coda/kernels/functional/qknorm_rope.py of the reference, implemented by coda_kernels_b200.functional.qknorm_rope."""

from coda_kernels_b200.functional.qknorm_rope import *  # noqa: F401,F403
from coda_kernels_b200.functional import qknorm_rope as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
