"""Paged state-tree KV cache: keys and values stored losslessly in 16-token pages of state-tree records (6400 B per
page per KV head against 8192 B in BF16), appended on write and read by the decode attention kernel without ever
being expanded.  PageStore holds one attention layer's pages (the tensors of the reference's statetree/kvcache.py
StateTreeKVLayer 49-57, with its append / dense / attention calls); PagedKVCache is the static cache of the decode
runner in this package.  The Hugging Face classes of the reference (StateTreeKVCache, StateTreeKVLayer,
statetree_attention, enable) live in hf_cache.py and are re-exported here when transformers is importable.
"""
import torch

from .ops import kv_ext

PAGE = 16
RKV = 1600


def decode_splits(B, Hkv, max_pages, sms=148, min_pages=4):
    """How many CTAs share each (sequence, KV head) of the decode attention kernel.  Two bounds: the split that
    balances a split's own pages against the cost of merging the partial results grows like the square root of the
    page count, and no more splits are needed than fill the GPU about three CTAs deep.  At least min_pages pages
    per split.  A function of the batch size and the longest context only, so one captured graph per batch size
    serves every step (the role of the reference's statetree/vllm_kv.py:42-50, re-sized for 148 SMs)."""
    by_length = int(round(max_pages ** 0.5))
    by_fill = -(-3 * sms // max(1, B * Hkv))
    most = max(1, max_pages // max(1, min_pages))
    return min(most, max(2, min(by_length, by_fill, 64)))               # two splits at least: several waves of CTAs


class PageStore:
    """pages of one attention layer: uint8 [blocks, H, 2, 2, 1600], escape pool int32 [P, 16], pool counter int32 [2]"""

    def __init__(self, num_blocks, num_kv_heads, device, pool_blocks=1 << 15):
        self.H = num_kv_heads
        self.device = torch.device(device)
        self.pages = torch.zeros(num_blocks, num_kv_heads, 2, 2, RKV, dtype=torch.uint8, device=device)
        self.pool = torch.zeros(pool_blocks, 16, dtype=torch.int32, device=device)
        self.pcnt = torch.zeros(2, dtype=torch.int32, device=device)
        self._wo = self._wml = None

    def append(self, K, V, slots, reuse=False):
        """K, V [N, H, 128] bf16 (heads contiguous), slots int64 [N] = block * 16 + row, -1 = padding token"""
        kv_ext().append(K, V, slots, self.pages, self.pool, self.pcnt, reuse)

    def attention(self, q, block_table, lens, scale, splits=1, starts=None, min_pages=1, out=None):
        """one query token per sequence: q [B, Hq, 128] bf16 -> [B, Hq, 128] bf16"""
        B, Hq, _ = q.shape
        if out is None:
            out = torch.empty(B, Hq, 128, dtype=torch.bfloat16, device=q.device)
        if splits > 1:
            need = B * Hq * splits
            if self._wo is None or self._wo.numel() < need * 128:
                self._wo = torch.empty(need * 128, dtype=torch.float32, device=q.device)
                self._wml = torch.empty(need * 2, dtype=torch.float32, device=q.device)
        else:
            if self._wo is None:
                self._wo = torch.empty(1, dtype=torch.float32, device=q.device)
                self._wml = torch.empty(1, dtype=torch.float32, device=q.device)
        kv_ext().attn(q, self.pages, self.pool, block_table, lens, out, self._wo, self._wml, scale, splits, starts,
                      min_pages)
        return out

    def dense(self, blocks=None):
        """pages (all, or the listed block ids) as exact BF16 Kd, Vd [n, 16, H, 128]"""
        n = self.pages.shape[0] if blocks is None else blocks.numel()
        Kd = torch.empty(n, PAGE, self.H, 128, dtype=torch.bfloat16, device=self.device)
        Vd = torch.empty_like(Kd)
        if blocks is None:
            kv_ext().dequant(self.pages, self.pool, Kd, Vd)
        else:
            kv_ext().dequant_blocks(self.pages, self.pool, blocks.to(torch.int32).contiguous(), Kd, Vd)
        return Kd, Vd

    def check(self):
        """raise if an escape could not be stored (extension pool exhausted): never silently lossy"""
        if int(self.pcnt[1].item()):
            raise RuntimeError("PagedKVCache: escape pool exhausted (pool_blocks too small)")

    def pool_usage(self):
        return int(self.pcnt[0].item()), self.pool.shape[0]


class PagedKVCache:
    """Static paged cache for a decoder: per-layer pages, one block table [B, max_pages] (sequence b owns pages
    b * max_pages ...), a GPU-side token count so decode steps are CUDA-graph safe."""

    def __init__(self, num_layers, batch_size, max_cache_len, num_kv_heads, device, pool_blocks=1 << 15):
        self.B = batch_size
        self.max_pages = (max_cache_len + PAGE - 1) // PAGE
        self.max_len = self.max_pages * PAGE
        self.device = torch.device(device)
        self.layers = [PageStore(batch_size * self.max_pages, num_kv_heads, device, pool_blocks)
                       for _ in range(num_layers)]
        self.bt32 = torch.arange(batch_size * self.max_pages, dtype=torch.int32, device=device).view(batch_size, -1)
        self.bt64 = self.bt32.long()
        self.lens = torch.zeros(batch_size, dtype=torch.int32, device=device)
        self.cum = torch.zeros((), dtype=torch.long, device=device)      # tokens stored (same for every sequence)
        self._stored = 0                                                  # the same count on the host, for capacity checks

    def update(self, layer_idx, key_states, value_states):
        """key/value_states [B, H, T, 128]; positions continue from the GPU-side count; returns the slots used"""
        B, H, T, D = key_states.shape
        self._stored += T if layer_idx == len(self.layers) - 1 else 0
        if self._stored + (T if layer_idx != len(self.layers) - 1 else 0) > self.max_len:
            raise ValueError(f"PagedKVCache.update: position {self._stored + T} exceeds the capacity of "
                             f"{self.max_len} tokens")
        cp = torch.arange(T, device=self.device) + self.cum
        slots = (self.bt64[:B][:, cp // PAGE] * PAGE + (cp % PAGE)).reshape(-1)
        K = key_states.transpose(1, 2).reshape(B * T, H, D)
        V = value_states.transpose(1, 2).reshape(B * T, H, D)
        self.layers[layer_idx].append(K.contiguous(), V.contiguous(), slots)
        if layer_idx == len(self.layers) - 1:
            self.cum += T
            self.lens[:B] = self.cum.to(torch.int32)
        elif layer_idx == 0:
            self.lens[:B] = (self.cum + T).to(torch.int32)
        return slots

    def begin_step(self, B):
        """decode step (one token per sequence): the slots every layer appends at, computed once; lens counts the new
        token.  Graph-safe (positions come from the GPU-side count)."""
        page = (self.cum // PAGE).clamp(max=self.max_pages - 1)            # a full cache never indexes past the table:
        slots = self.bt64[:B].gather(1, page.expand(B, 1)).view(B) * PAGE + self.cum % PAGE
        slots = torch.where(self.cum < self.max_len, slots, torch.full_like(slots, -1))   # ... the token is dropped
        self.lens[:B] = (self.cum + 1).clamp(max=self.max_len).to(torch.int32)
        return slots

    def end_step(self):
        self.cum += 1

    def attention(self, layer_idx, q, scale, splits=None):
        """decode step: q [B, Hq, 128] against everything stored in the layer (including this step's token)"""
        B = q.shape[0]
        if splits is None:
            splits = decode_splits(B, self.layers[layer_idx].H, self.max_pages)
        return self.layers[layer_idx].attention(q, self.bt32[:B], self.lens[:B], scale, splits, None, 4)

    def check(self):
        for layer in self.layers:
            layer.check()

    def reset(self):
        self._stored = 0
        self.cum.zero_()
        self.lens.zero_()
        for layer in self.layers:
            layer.pcnt.zero_()


try:                                                   # the transformers glue, under the reference's names
    from .hf_cache import StateTreeKVCache, StateTreeKVLayer, enable, statetree_attention  # noqa: E402,F401
except ImportError:                                    # transformers absent or too old: the page store still works
    pass
