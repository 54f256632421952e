"""Same public names as coda/kernels/blocks/llama3.py of the reference, implemented by ``coda_kernels_b200.blocks.llama3``."""

from coda_kernels_b200.blocks.llama3 import (  # noqa: F401
    Block,
    BlockPost,
    BlockPre,
    block,
    block_backward,
    block_forward,
    block_post,
    block_post_backward,
    block_post_forward,
    block_pre,
    block_pre_backward,
    block_pre_forward,
)
