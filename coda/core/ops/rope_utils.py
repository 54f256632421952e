"""``make_rope_frequencies`` under the module path the reference's benchmarks import (benchmarks/utils/operands.py:10)."""

from coda_kernels_b200.rope_utils import make_rope_frequencies, rope_inv_freq

__all__ = ["make_rope_frequencies", "rope_inv_freq"]
