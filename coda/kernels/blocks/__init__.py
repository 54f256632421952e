"""``coda.kernels.blocks`` of the drop-in layout: the fused Llama-3 layer blocks."""
