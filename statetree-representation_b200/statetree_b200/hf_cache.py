"""Hugging Face transformers glue for the compressed KV pages: a `Cache` whose layers keep keys and values in
state-tree pages, and the `statetree` attention function that serves decode steps (one new token per sequence)
straight from those pages and leaves everything else (prefill) to SDPA.  Same names and call order as the reference's
statetree/kvcache.py (StateTreeKVLayer 35-129, StateTreeKVCache 132-177, statetree_attention 180-201, enable 204-213):

    from statetree_b200.kvcache import StateTreeKVCache, enable
    enable(model)
    cache = StateTreeKVCache(model.config, batch_size=B, max_cache_len=prompt + new)
    model.generate(input_ids, attention_mask=mask, past_key_values=cache, max_new_tokens=new)

Positions come from a GPU-side token count (or from `cache_position` when the model passes it), buffers are static,
so decode steps can be captured in CUDA graphs.  Left padding is supported: each sequence's first valid position is
read once from the prefill attention mask.  Head dimension 128 only.
"""
import threading

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from .kvcache import PAGE, PageStore, decode_splits

_LAST = threading.local()          # the layer whose update() ran last on this thread; the attention function picks it up


class StateTreeKVLayer(CacheLayerMixin):
    """one attention layer's pages inside a StateTreeKVCache"""
    is_compileable = False
    is_sliding = False

    def __init__(self, cache, layer_idx):
        super().__init__()
        self.cache, self.layer_idx = cache, layer_idx
        self.store = None
        self.host_len = 0                            # tokens stored, counted on the host (eager generate, prefill)
        self.max_cache_len = cache.max_len
        self.max_batch_size = cache.alloc_batch

    def lazy_initialization(self, key_states, value_states=None):
        c = self.cache
        B, H, _, D = key_states.shape
        if D != 128:
            raise ValueError("StateTreeKVCache: the page format holds heads of dimension 128")
        c._allocate(B, H, key_states.device)
        self.dtype, self.device = key_states.dtype, key_states.device
        self.num_heads = H
        self.max_batch_size = self.batch_size = c.Bmax
        self.store = PageStore(c.Bmax * c.max_pages, H, self.device, pool_blocks=c.pool_blocks)
        self.gpu_len = torch.zeros((), dtype=torch.long, device=self.device)     # the same count on the GPU (graphs)
        self.is_initialized = True

    @property
    def pages(self):
        return self.store.pages

    def update(self, key_states, value_states, *args, **kwargs):
        opts = args[0] if args else kwargs.get("cache_kwargs")
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        c = self.cache
        B, H, T, D = key_states.shape
        where = opts.get("cache_position") if isinstance(opts, dict) else None
        if where is None:
            where = self.gpu_len + torch.arange(T, device=self.device)
        self.gpu_len.copy_(where[-1] + 1)
        slots = (c.table64[:B].index_select(1, where // PAGE) * PAGE + where % PAGE).reshape(-1)
        rows = []
        for t in (key_states, value_states):
            t = t.transpose(1, 2).reshape(B * T, H, D)
            rows.append(t if (t.stride(2) == 1 and t.stride(1) == D) else t.contiguous())
        self.store.append(rows[0], rows[1], slots)
        _LAST.layer = self
        before, self.host_len = self.host_len, self.host_len + T
        if T == 1:                                   # a decode step: the attention function reads the pages itself
            if self.layer_idx == 0:
                c.lens[:B].copy_((where[-1:] + 1).to(torch.int32).expand(B))
            return key_states, value_states
        if before == 0:                              # first prefill chunk: attention over the prompt's own K / V
            return key_states, value_states
        old_k, old_v = self.dense(before)            # a later chunk attends to the stored prefix too
        return torch.cat([old_k, key_states], 2), torch.cat([old_v, value_states], 2)

    def dense(self, n):
        """the first n stored tokens of every sequence as exact BF16 [B, H, n, 128]"""
        c = self.cache
        pos = torch.arange(n, device=self.device)
        blocks = c.table64[:c.Bmax].index_select(1, pos // PAGE)                # [B, n]
        Kd, Vd = self.store.dense()
        row = (pos % PAGE).unsqueeze(0).expand_as(blocks)
        return Kd[blocks, row].transpose(1, 2), Vd[blocks, row].transpose(1, 2)

    def get_mask_sizes(self, query_length, *args, **kwargs):
        q = query_length.shape[0] if isinstance(query_length, torch.Tensor) else int(query_length)
        return self.host_len + q, 0

    def get_seq_length(self, *args, **kwargs):
        return self.gpu_len if self.is_initialized else 0

    def get_max_cache_shape(self):
        return self.max_cache_len

    get_max_length = get_max_cache_shape                   # the name older Transformers releases call

    get_max_length = get_max_cache_shape

    def reset(self):
        self.host_len = 0
        if self.is_initialized:
            self.store.pcnt.zero_()
            self.gpu_len.zero_()
        self.cache.starts_known = False

    def check(self):
        if self.is_initialized:
            self.store.check()

    def reorder_cache(self, beam_idx):
        raise NotImplementedError("StateTreeKVCache: beam search is not supported")

    def crop(self, max_length):
        raise NotImplementedError("StateTreeKVCache: crop is not supported")


class StateTreeKVCache(Cache):
    """Lossless compressed KV cache for transformers models.  batch_size and max_cache_len fix the page tables;
    pool_blocks sizes each layer's pool of 64-byte escape extension blocks."""

    def __init__(self, config, batch_size=None, max_cache_len=4096, pool_blocks=None, **kwargs):
        text = config.get_text_config() if hasattr(config, "get_text_config") else config
        self.num_layers = text.num_hidden_layers
        self.num_q_heads = text.num_attention_heads
        self.num_kv_heads = getattr(text, "num_key_value_heads", None) or text.num_attention_heads
        self.max_len = int(max_cache_len)
        self.max_pages = -(-self.max_len // PAGE)
        self.alloc_batch, self.pool_blocks = batch_size, pool_blocks
        self.starts_known = False
        self._allocated = False
        super().__init__(layers=[StateTreeKVLayer(self, i) for i in range(self.num_layers)])

    def _allocate(self, B, H, device):
        if self._allocated:
            if B > self.Bmax:
                raise ValueError(f"StateTreeKVCache: batch {B} is larger than the {self.Bmax} sequences it was sized for")
            return
        self.Bmax = max(B, self.alloc_batch or 0)
        n = self.Bmax
        self.table64 = torch.arange(n * self.max_pages, device=device).view(n, self.max_pages)
        self.table32 = self.table64.to(torch.int32)
        self.lens = torch.zeros(n, dtype=torch.int32, device=device)
        self.starts = torch.zeros(n, dtype=torch.int32, device=device)
        self.splits = decode_splits(n, H, self.max_pages)
        if self.pool_blocks is None:
            self.pool_blocks = max(4096, n * self.max_pages * H * 4 // 8)
        self._allocated = True

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None, *args, **kwargs):
        return self.layers[layer_idx].update(key_states, value_states, cache_kwargs)

    def check(self):
        """raise if an escape could not be stored anywhere (pool too small): the cache is never silently lossy"""
        for layer in self.layers:
            layer.check()

    def storage_bytes(self):
        return sum(l.store.pages.numel() + l.store.pool.numel() * 4 for l in self.layers if l.is_initialized)


def statetree_attention(module, query, key, value, attention_mask, dropout=0.0, scaling=None, **kwargs):
    """the 'statetree' attention implementation: a decode step reads the compressed pages, anything else runs SDPA"""
    from transformers.integrations.sdpa_attention import sdpa_attention_forward
    layer = getattr(_LAST, "layer", None)
    _LAST.layer = None
    if layer is not None and layer.layer_idx == getattr(module, "layer_idx", layer.layer_idx):
        c = layer.cache
        B, Hq, T, D = query.shape
        if T == 1 and layer.host_len > 1:
            q = query[:, :, 0, :]
            if q.stride(-1) != 1 or q.stride(1) != D:
                q = q.contiguous()
            scale = float(scaling) if scaling is not None else D ** -0.5
            out = layer.store.attention(q, c.table32[:B], c.lens[:B], scale, splits=c.splits, starts=c.starts[:B],
                                        min_pages=4)
            return out.view(B, 1, Hq, D), None
        if T > 1 and not c.starts_known and attention_mask is not None and attention_mask.dim() == 4:
            last_row = attention_mask[:, 0, -1, :]                  # the last query sees everything but the padding
            masked = ~last_row if last_row.dtype == torch.bool else last_row < 0
            c.starts[:B].copy_(masked.sum(-1).to(torch.int32))
            c.starts_known = True
    return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling, **kwargs)


def enable(model):
    """register the 'statetree' attention implementation and switch `model` to it (use with a StateTreeKVCache)"""
    from transformers import AttentionInterface
    from transformers.masking_utils import AttentionMaskInterface, sdpa_mask
    AttentionInterface.register("statetree", statetree_attention)
    AttentionMaskInterface.register("statetree", sdpa_mask)
    if hasattr(model, "set_attn_implementation"):
        model.set_attn_implementation("statetree")
    else:
        model.config._attn_implementation = "statetree"
    return model
