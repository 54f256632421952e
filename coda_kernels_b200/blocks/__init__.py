"""Fused whole-layer blocks built from the GEMM + epilogue operators (counterpart of ``coda.kernels.blocks``)."""

from . import llama3

__all__ = ["llama3"]
