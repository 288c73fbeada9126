"""statetree_b200: the state-tree decode hot path (lossless ~12-bit BF16 weights and KV pages) on NVIDIA B200.

Same Python surface as the reference package for this path (format.encode / decode_reference, TreeLinear / TreeSlice /
TreeEmbedding, the MoE wrappers and TreeExperts, the paged KV cache), over hand-written sm_100a CUDA kernels behind a
C ABI (include/statetree_b200.h).  CUDA only: there is no CPU or eager fallback.
"""
from .format import decode_reference, encode  # noqa: F401
from .experts import TreeExperts  # noqa: F401
from .linear import TreeEmbedding, TreeLinear, TreeSlice  # noqa: F401
from .model import (DEFAULT_FUSE, convert, load_pretrained, prepare, save_pretrained, size_report,  # noqa: F401
                    tree_modules)

__version__ = "0.2.0"
# the names the reference package exports (statetree/__init__.py:10-17), so that `import statetree_b200 as statetree`
# keeps a caller's convert / prepare / save_pretrained / load_pretrained lines as they are
__all__ = ["TreeLinear", "TreeSlice", "TreeEmbedding", "TreeExperts", "DEFAULT_FUSE", "convert", "prepare",
           "save_pretrained", "load_pretrained", "size_report", "tree_modules", "encode", "decode_reference"]
