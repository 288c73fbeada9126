"""Module object with the names and signatures of the reference's `statetree._kv` extension
(statetree/csrc/kvcache.cu:588-599): append, dequant, dequant_blocks, attn, page_bytes, version.  Code written against
`statetree.ops.kv_ext()` can be pointed here unchanged; every call goes through the C ABI of libstatetree_b200.so.
"""
from .ops import _KV as _impl
from .ops import lib as _lib

_lib()                                   # fail at import time, loudly, when the kernel library has not been built

append = _impl.append
dequant = _impl.dequant
dequant_blocks = _impl.dequant_blocks
attn = _impl.attn
page_bytes = _impl.page_bytes
version = _impl.version
