"""The parts of the reference's vLLM KV-cache backend (statetree/vllm_kv.py, written against vLLM 0.32) that do not
need vLLM itself: the page specification, the decode split contract, the per-process escape pool with its delayed
exhaustion check, the view of a vLLM layer cache as pages, and a `PageBackend` that performs the three data-path
calls of the backend (write at a slot mapping with recycling, decode attention over the pages, exact decode of cached
prefix pages for a paged prefill kernel).  The vLLM-facing classes (AttentionBackend / metadata builder / impl) are
thin wrappers over these; they are not built here because this image ships vLLM 0.22, whose v1 attention interface
differs ("vLLM 0.32 absent"): `register()` reports that instead of installing anything.
"""
import os

import torch

from .kvcache import decode_splits as _splits_for_pages
from .ops import kv_ext

PAGE, RKV, HD = 16, 1600, 128
BYTES_PER_TOKEN_PER_HEAD = 4 * RKV // PAGE           # 400 (BF16: 512): what the backend declares to the block manager
MIN_PAGES_PER_SPLIT = 4
MAX_SPLITS = 32


def decode_splits(num_decodes, num_kv_heads, sms=148):
    """Split count of a decode batch as a function of the (padded) batch size only, so the CUDA graph captured for a
    batch size serves every context length: the kernel keeps at least MIN_PAGES_PER_SPLIT pages per split and idle
    splits exit at once.  A power of two, at most MAX_SPLITS (contract of statetree/vllm_kv.py:42-50, sized for a GPU
    of `sms` SMs running about three CTAs each)."""
    if num_decodes <= 0:
        return 1
    want = (3 * sms) // (num_decodes * num_kv_heads)
    if want <= 1:
        return 1
    return 1 << (min(want, MAX_SPLITS).bit_length() - 1)


def page_view(kv_cache, num_kv_heads):
    """a vLLM layer cache [blocks, H, 16, 400 B] (any dtype of the right size) as the kernels' uint8
    [blocks, H, 2, 2, 1600]"""
    raw = kv_cache if kv_cache.dtype == torch.uint8 else kv_cache.view(torch.uint8)
    blocks = raw.shape[0]
    if not raw.is_contiguous() or raw.numel() != blocks * num_kv_heads * 4 * RKV:
        raise RuntimeError(f"statetree KV: unexpected layer cache {tuple(kv_cache.shape)} / strides {kv_cache.stride()}")
    return raw.view(blocks, num_kv_heads, 2, 2, RKV)


class SharedPool:
    """One per process and device: the escape extension pool shared by all layers, the split workspace, and a watch on
    the pool counters.  poll() runs once per step on the host and looks at the counters copied at the PREVIOUS step,
    so it never synchronises; exhaustion therefore raises one step late, but it always raises (never silently lossy)."""

    def __init__(self, device, num_q_heads, num_kv_heads, pool_mb=None, max_rows=None):
        mb = float(os.environ.get("STATETREE_KV_POOL_MB", "128")) if pool_mb is None else float(pool_mb)
        blocks = min(max(1024, int(mb * 2 ** 20) // 64), (1 << 23) - 1)
        self.device = torch.device(device)
        self.pool = torch.zeros(blocks, 16, dtype=torch.int32, device=self.device)
        self.cnt = torch.zeros(2, dtype=torch.int32, device=self.device)      # [0] blocks handed out, [1] exhausted
        self.host = torch.zeros(2, dtype=torch.int32)
        if self.device.type == "cuda":
            self.host = self.host.pin_memory()
        self.num_q_heads, self.num_kv_heads = num_q_heads, num_kv_heads
        rows = max_rows or max((3 * 148) // num_kv_heads, MAX_SPLITS)          # >= batch x splits for every batch size
        self.wo = torch.empty(rows * num_q_heads * HD, dtype=torch.float32, device=self.device)
        self.wml = torch.empty(rows * num_q_heads * 2, dtype=torch.float32, device=self.device)
        self.steps, self.warned = 0, False

    def poll(self):
        if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
            return None
        used, exhausted = int(self.host[0]), int(self.host[1])
        if exhausted:
            raise RuntimeError(f"statetree KV: the escape extension pool ({self.pool.shape[0]} blocks) is exhausted; "
                               "restart with a larger STATETREE_KV_POOL_MB")
        self.steps += 1
        note = None
        if not self.warned and used > 0.5 * self.pool.shape[0]:
            self.warned = True
            note = f"statetree KV: extension pool {100 * used / self.pool.shape[0]:.0f}% used ({used} blocks)"
        self.host.copy_(self.cnt, non_blocking=True)
        return note

    def usage(self):
        """(blocks used, blocks, exhausted); synchronises (for tests and diagnostics)"""
        used, exhausted = self.cnt.tolist()
        return used, self.pool.shape[0], bool(exhausted)


_POOLS = {}


def shared_pool(device, num_q_heads, num_kv_heads):
    """the process's SharedPool of a device, made on first use (one pool serves every layer of a model, so all layers
    must have the same head counts; reference: statetree/vllm_kv.py:88-98)"""
    device = torch.device(device)
    key = (device.type, device.index)
    pool = _POOLS.get(key)
    if pool is None:
        pool = _POOLS[key] = SharedPool(device, num_q_heads, num_kv_heads)
    elif (pool.num_q_heads, pool.num_kv_heads) != (num_q_heads, num_kv_heads):
        raise NotImplementedError("statetree KV: layers with different head counts in one model")
    return pool


def pool_usage():
    """{(device type, index): (blocks used, blocks, exhausted)} of this process's pools; synchronises (for tests;
    reference: statetree/vllm_kv.py:101-107)"""
    return {key: pool.usage() for key, pool in _POOLS.items()}


class PageBackend:
    """The data path of the vLLM backend for one attention layer configuration (reference: StateTreeKVImpl,
    statetree/vllm_kv.py:228-318): write, decode, and the exact decode of cached pages for prefill."""

    def __init__(self, num_heads, num_kv_heads, scale, shared):
        if num_heads % num_kv_heads or num_heads // num_kv_heads > 8:
            raise NotImplementedError("statetree KV: at most 8 query heads per KV head")
        self.num_heads, self.num_kv_heads, self.scale, self.shared = num_heads, num_kv_heads, float(scale), shared
        self.kx = kv_ext()

    def write(self, key, value, kv_cache, slot_mapping):
        """do_kv_cache_update: append at vLLM's slot mapping; a block that is written from its first row again
        recycles its extension chain (reuse=True), so the shared pool does not leak across requests"""
        n = slot_mapping.shape[0]
        if n <= 0 or kv_cache.numel() == 0:
            return
        k = key[:n].view(n, self.num_kv_heads, HD)
        v = value[:n].view(n, self.num_kv_heads, HD)
        self.kx.append(k, v, slot_mapping[:n], page_view(kv_cache, self.num_kv_heads), self.shared.pool, self.shared.cnt,
                       True)

    def decode(self, query, kv_cache, block_table, seq_lens, out, splits=None):
        """one query token per request: attention straight from the pages into out [n, Hq, 128]"""
        n = query.shape[0]
        if splits is None:
            splits = decode_splits(n, self.num_kv_heads)
        self.kx.attn(query.view(n, self.num_heads, HD), page_view(kv_cache, self.num_kv_heads), self.shared.pool,
                     block_table[:n], seq_lens[:n], out.view(n, self.num_heads, HD), self.shared.wo, self.shared.wml,
                     self.scale, splits, None, MIN_PAGES_PER_SPLIT)
        return out

    def cached_pages(self, kv_cache, blocks):
        """requests with cached context (prefix caching, chunked prefill): the listed cache blocks decoded exactly into
        BF16 scratch pages Kd, Vd [n, 16, Hkv, 128] that a paged prefill attention kernel can read"""
        n = blocks.numel()
        pages = page_view(kv_cache, self.num_kv_heads)
        Kd = torch.empty(n, PAGE, self.num_kv_heads, HD, dtype=torch.bfloat16, device=pages.device)
        Vd = torch.empty_like(Kd)
        self.kx.dequant_blocks(pages, self.shared.pool, blocks.to(torch.int32).contiguous(), Kd, Vd)
        return Kd, Vd


def prefill_page_tables(seq_lens, block_table, first_request=0):
    """For prefill requests with cached context: which cache block backs scratch page i, and each request's scratch
    block table (host arithmetic of statetree/vllm_kv.py:208-225).  seq_lens: int64 CPU tensor [requests] (cached + new
    tokens); block_table: [all requests, max blocks] on the device.  Returns (blocks int32 [pages] on the device,
    scratch table int32 [requests, max pages] on the device)."""
    pages = (seq_lens + PAGE - 1) // PAGE
    total = int(pages.sum())
    first = torch.cumsum(pages, 0) - pages
    req = torch.repeat_interleave(torch.arange(seq_lens.numel()), pages)
    page = torch.arange(total) - torch.repeat_interleave(first, pages)
    table = torch.zeros(seq_lens.numel(), int(pages.max()), dtype=torch.int32)
    table[req, page] = torch.arange(total, dtype=torch.int32)
    dev = block_table.device
    blocks = block_table[(req + first_request).to(dev), page.to(dev)].to(torch.int32).contiguous()
    return blocks, table.to(dev)


def register():
    """What the reference's vLLM plugin does at import (statetree/vllm_plugin.py:36-46) needs vLLM 0.32's v1 attention
    interface.  Returns (installed, reason)."""
    try:
        import vllm
    except ImportError:
        return False, "vLLM is not installed"
    version = getattr(vllm, "__version__", "0")
    try:
        from vllm.v1.attention.backend import AttentionBackend  # noqa: F401
        from vllm.v1.kv_cache_layout import KVCacheLayout  # noqa: F401
    except ImportError:
        return False, f"vLLM {version} does not have the 0.32 attention-backend interface this backend targets"
    return False, f"vLLM {version}: the backend classes are not built in this package (data path: PageBackend)"
