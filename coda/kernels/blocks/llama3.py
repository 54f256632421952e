"""Same public names as coda/kernels/blocks/llama3.py of the reference, implemented by ``coda_kernels_b200.blocks.llama3``."""

from coda_kernels_b200.blocks.llama3 import Block, BlockPost, BlockPre, block, block_post, block_pre  # noqa: F401
