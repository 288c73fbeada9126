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


def install_as(name="statetree"):
    """Make `import <name>` resolve to this package, submodules included (`<name>.format`, `.linear`, `.experts`,
    `.model`, `.kvcache`, `.ops`, `.vllm_kv`, `._kv`, and `._vllm` for the vLLM layer methods), so that code written
    against the reference package runs unchanged:

        import statetree_b200; statetree_b200.install_as("statetree")
        import statetree; from statetree.linear import TreeLinear; statetree.ops.ext()

    Refuses to replace a different module that is already imported under that name."""
    import importlib
    import sys
    me = sys.modules[__name__]
    have = sys.modules.get(name)
    if have is not None and have is not me:
        raise RuntimeError(f"install_as: another module is already imported as {name!r} ({getattr(have, '__file__', '?')})")
    sys.modules[name] = me
    aliases = {"format": "format", "linear": "linear", "experts": "experts", "model": "model", "kvcache": "kvcache",
               "ops": "ops", "vllm_kv": "vllm_kv", "_kv": "_kv", "_vllm": "vllm_layers"}
    for theirs, mine in aliases.items():
        sys.modules[f"{name}.{theirs}"] = importlib.import_module(f"{__name__}.{mine}")
    return me
