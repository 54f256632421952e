"""``coda.core.gemm`` of the drop-in layout: the GEMM + epilogue operators under the reference's names."""
