"""statetree_b200: the state-tree decode hot path (lossless ~12-bit BF16 weights and KV pages) on NVIDIA B200.

Same Python surface as the reference package for this path (format.encode / decode_reference, TreeLinear / TreeSlice /
TreeEmbedding, the MoE wrappers and TreeExperts, the paged KV cache), over hand-written sm_100a CUDA kernels behind a
C ABI (include/statetree_b200.h).  CUDA only: there is no CPU or eager fallback.
"""
from .format import decode_reference, encode  # noqa: F401
from .linear import TreeEmbedding, TreeLinear, TreeSlice  # noqa: F401

__version__ = "0.1.0"
__all__ = ["TreeLinear", "TreeSlice", "TreeEmbedding", "encode", "decode_reference"]
