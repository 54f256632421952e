"""``CodaRuntime`` of the reference's TorchTitan integration (benchmarks/torchtitan/llama3_coda.py), bound to the B200 blocks."""

from coda_kernels_b200.blocks.runtime import CodaRuntime, Llama3Runtime  # noqa: F401
