"""A minimal Qwen3-architecture decoder over the tree-stored layers, for decode-throughput measurement with random
weights: RMSNorm, fused q/k/v and gate/up projections, per-head q/k RMSNorm, RoPE, grouped-query attention over the
compressed KV pages, SwiGLU, untied lm_head, greedy sampling.  One decode step is captured in a CUDA graph and
replayed (the measurement method of the reference's statetree/bench.py:74-133 DecodeRunner).  `compressed=False`
builds the BF16 control from the same seeds: dense weights, a dense BF16 KV cache and FlashAttention.

Tensor parallelism (one process per GPU): q/k/v and gate/up are split by rows (heads / intermediate columns), o and
down by input columns with an all-reduce of their outputs, the lm_head by vocabulary rows with an all-gather of the
logits; embeddings and norms are replicated.  With `experts > 0` the MLP is a routed expert block (softmax router,
top-k, renormalised weights, TreeExperts): under several ranks the attention stays tensor-parallel and the experts are
split over the ranks (expert parallelism: every rank routes all tokens, computes its own experts' weighted partial
output, and the partial outputs are all-reduced).  Every rank draws the full tensors from the same seeds and keeps its slice,
so a tensor-parallel run computes the same function as the single-GPU one.
"""
import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as Fn

from .kvcache import PagedKVCache
from .linear import TreeLinear, interleave_gate_up
from .ops import ext, kv_ext


def _flash():
    from flash_attn import flash_attn_with_kvcache
    return flash_attn_with_kvcache


@dataclass
class DecoderConfig:
    layers: int = 36
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    inter: int = 12288
    vocab: int = 151936
    rope_theta: float = 1e6
    eps: float = 1e-6
    experts: int = 0                 # > 0: the MLP of every layer is a routed mixture of experts (Qwen3-MoE shape)
    top_k: int = 8
    moe_inter: int = 768             # intermediate size of one expert
    distinct_experts: int = 4        # random expert matrices drawn per layer; the others are copies in their own buffers


class _Dense:
    """BF16 control for a TreeLinear: same call, dense weight"""

    def __init__(self, W):
        self.W = W
        self.out_features, self.in_features = W.shape

    def __call__(self, x):
        return Fn.linear(x, self.W)

    def record_bytes(self):
        return self.W.numel() * 2


class TreeDecoder:
    def __init__(self, cfg, device, batch, max_len, compressed=True, seed=0, rank=0, world=1, group=None):
        self.cfg, self.dev, self.B, self.rank, self.world, self.group = cfg, torch.device(device), batch, rank, world, group
        self.compressed = compressed
        c = cfg
        assert c.heads % world == 0 and c.kv_heads % world == 0 and c.inter % (64 * world) == 0 and c.vocab % (16 * world) == 0
        self.hq, self.hkv = c.heads // world, c.kv_heads // world
        self.fused_act = False
        if c.experts:
            assert compressed, "the mixture-of-experts decoder has no BF16 control"
            assert c.experts % world == 0
            from .parallel import expert_partition
            self.e_lo, self.e_hi, self.emap = expert_partition(c.experts, rank, world, self.dev)
        if compressed and not c.experts and batch <= 8:
            from .ops import lib
            with torch.cuda.device(self.dev):
                self.fused_act = bool(lib().st_gemv_swiglu_supported(2 * c.inter // world, c.hidden, batch))
        gen = torch.Generator(device=self.dev)
        self._tid = 0

        def draw(rows, cols):
            gen.manual_seed(seed * 100003 + self._tid)
            self._tid += 1
            return (torch.randn(rows, cols, device=self.dev, generator=gen) * 0.02).to(torch.bfloat16)

        def make(W):
            return TreeLinear.from_weight(W.contiguous(), verify=False) if compressed else _Dense(W.contiguous())

        def rows(W, n_parts=1):
            per = W.shape[0] // world
            return W[rank * per:(rank + 1) * per]

        D = c.head_dim
        self.embed = make(draw(c.vocab, c.hidden))
        self.blocks = []
        for _ in range(c.layers):
            q, k, v = draw(c.heads * D, c.hidden), draw(c.kv_heads * D, c.hidden), draw(c.kv_heads * D, c.hidden)
            qkv = make(torch.cat([rows(q), rows(k), rows(v)]))
            del q, k, v
            o = draw(c.hidden, c.heads * D)
            per = o.shape[1] // world
            o = make(o[:, rank * per:(rank + 1) * per])
            if c.experts:
                gu, d = self._make_experts(draw), None
            else:
                g, u = draw(c.inter, c.hidden), draw(c.inter, c.hidden)
                if self.fused_act:                          # gate / up tiles in turn: SwiGLU in the GEMV's epilogue
                    gu = make(interleave_gate_up(rows(g).contiguous(), rows(u).contiguous()))
                else:
                    gu = make(torch.cat([rows(g), rows(u)]))
                del g, u
                d = draw(c.hidden, c.inter)
                per = d.shape[1] // world
                d = make(d[:, rank * per:(rank + 1) * per])
            self.blocks.append((qkv, o, gu, d))
        self.lm_head = make(rows(draw(c.vocab, c.hidden)))
        ones = torch.ones(c.hidden, dtype=torch.bfloat16, device=self.dev)
        self.norm_w, self.head_norm_w = ones, torch.ones(D, dtype=torch.bfloat16, device=self.dev)
        # rotary tables
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, D, 2, device=self.dev, dtype=torch.float32) / D))
        ang = torch.arange(max_len, device=self.dev, dtype=torch.float32)[:, None] * inv[None]
        self.cos, self.sin = ang.cos().contiguous(), ang.sin().contiguous()      # float32 [max_len, 64]
        self.max_len = max_len
        self.pos_buf = torch.zeros(1, dtype=torch.long, device=self.dev)
        self.h_buf = torch.empty(batch, c.hidden, dtype=torch.bfloat16, device=self.dev)
        self.q_buf = torch.empty(batch, self.hq, D, dtype=torch.bfloat16, device=self.dev)
        self.k_buf = torch.empty(batch, self.hkv, D, dtype=torch.bfloat16, device=self.dev)
        self.tokens = torch.zeros(batch, dtype=torch.long, device=self.dev)
        if compressed:
            self.cache = PagedKVCache(c.layers, batch, max_len, self.hkv, self.dev, pool_blocks=1 << 14)
        else:
            self.kc = [torch.zeros(batch, max_len, self.hkv, D, dtype=torch.bfloat16, device=self.dev) for _ in range(c.layers)]
            self.vc = [torch.zeros_like(k) for k in self.kc]
            self.lens = torch.zeros(batch, dtype=torch.int32, device=self.dev)
        self.comm = None
        if world > 1 and batch <= 64 and c.hidden <= 8192 and c.hidden % 8 == 0:
            from .parallel import peer_comm
            self.comm = peer_comm(group)
        self.graph = None
        # RMSNorm(x + delta) formed inside the GEMV that consumes it (no add + norm launch in front of q/k/v, gate/up
        # and the output head) where the kernel takes the shape
        self.pre_qkv = self.pre_gu = self.pre_head = False
        if compressed and batch <= 8:
            E = ext()
            qkv0, _, gu0, _ = self.blocks[0]
            with torch.cuda.device(self.dev):
                self.pre_qkv = E.gemv_prenorm_supported(qkv0.out_features, c.hidden, batch, False)
                self.pre_gu = (not c.experts) and E.gemv_prenorm_supported(gu0.out_features, c.hidden, batch, self.fused_act)
                self.pre_head = E.gemv_prenorm_supported(self.lm_head.out_features, c.hidden, batch, False)
            self._xbuf = [torch.empty(batch, c.hidden, dtype=torch.bfloat16, device=self.dev) for _ in range(2)]

    def _prenorm_linear(self, layer, x, delta, act=False):
        """(layer(RMSNorm(x + delta) * w), x + delta) in one launch; the new residual stream goes to the buffer x is not in"""
        from .linear import _state
        E = ext()
        B, M, N = x.shape[0], layer.out_features, layer.in_features
        eo, el, eb = layer.tables()
        y = torch.empty(B, M // 2 if act else M, dtype=torch.bfloat16, device=self.dev)
        x_out = None
        if delta is not None:
            x_out = self._xbuf[1] if x is self._xbuf[0] else self._xbuf[0]
        ws = _state(self.dev).get_ws(E.gemv_workspace_bytes(M, N, B))
        E.gemv_prenorm(layer.tree, eo, eb, el, x, delta, self.norm_w, self.cfg.eps, x_out, y, ws, act)
        return y, (x if x_out is None else x_out)

    def _make_experts(self, draw):
        """(router weight [E, hidden] BF16, TreeExperts over this rank's experts): `distinct_experts` random matrices per
        projection, every expert a copy of one of them in a buffer of its own (so the records of every expert a step
        touches stream from HBM), which keeps building a 128-expert x 48-layer model within minutes"""
        from .experts import TreeExperts
        c = self.cfg
        router = draw(c.experts, c.hidden)
        base13 = [TreeLinear.from_weight(draw(2 * c.moe_inter, c.hidden), verify=False) for _ in range(c.distinct_experts)]
        base2 = [TreeLinear.from_weight(draw(c.hidden, c.moe_inter), verify=False) for _ in range(c.distinct_experts)]

        def copy_of(tl):
            m = TreeLinear(tl.in_features, tl.out_features, device="meta", n_esc=tl.esc_rows.numel())
            m._buffers["tree"] = tl.tree.clone()
            for k in ("esc_rows", "esc_cols", "esc_bits"):
                m._buffers[k] = tl._buffers[k]
            m._tables = tl.tables()
            return m

        mine = range(self.e_lo, self.e_hi)
        te = TreeExperts([copy_of(base13[e % c.distinct_experts]) for e in mine],
                         [copy_of(base2[e % c.distinct_experts]) for e in mine])
        te.tables()
        return (router, te)

    def weight_bytes(self):
        """record bytes a decode step reads on this rank (the embedding table is read B rows at a time; of the experts,
        an upper bound: min(experts on the rank, batch x top_k) of them)"""
        n = self.lm_head.record_bytes()
        for qkv, o, gu, d in self.blocks:
            n += qkv.record_bytes() + o.record_bytes()
            if self.cfg.experts:
                te = gu[1]
                per = te.record_bytes() // te.num_experts
                n += per * min(te.num_experts, self.B * self.cfg.top_k)
            else:
                n += gu.record_bytes() + d.record_bytes()
        return n

    def _row_parallel(self, layer, xin):
        """(delta, summed): the output of a row-parallel projection (o, down) on this rank's activation slice.  A tree
        layer at GEMV batch sizes sums over the ranks inside its own kernel (summed = True); otherwise the partial
        output comes back and _add_norm adds the ranks."""
        from .linear import GEMV_MAX, _state
        B = xin.shape[0]
        if (self.world > 1 and self.comm is not None and self.compressed and B <= min(GEMV_MAX, 32)
                and layer.bias is None and self.comm.gemv_allreduce_fits(layer.out_features, B)):
            eo, el, eb = layer.tables()
            y = torch.empty(B, layer.out_features, dtype=torch.bfloat16, device=self.dev)
            ws = _state(self.dev).get_ws(ext().gemv_workspace_bytes(layer.out_features, layer.in_features, B))
            self.comm.gemv_allreduce(layer.tree, eo, eb, el, xin, y, ws)
            return y, True
        return layer(xin), False

    def _add_norm(self, x, delta, h, summed=False):
        """x += (all-reduced) delta; h = RMSNorm(x) * w.  Under tensor parallelism delta is this rank's partial output of
        a row-parallel projection unless `summed`: one kernel sums it over the ranks through peer memory and applies
        add + norm."""
        c = self.cfg
        if delta is not None and self.world > 1 and not summed:
            if self.comm is not None:
                self.comm.all_reduce_add_rmsnorm(x, delta, self.norm_w, h, c.eps)
                return
            dist.all_reduce(delta, group=self.group)
        ext().add_rmsnorm(x, delta, self.norm_w, h, c.eps)

    def _step(self):
        """one decode step for self.tokens at position self.pos; about ten launches per layer"""
        c, B, D = self.cfg, self.B, self.cfg.head_dim
        E = ext()
        x = self.embed.rows(self.tokens) if self.compressed else self.embed.W[self.tokens]
        scale = 1.0 / math.sqrt(D)
        h, qb, kb = self.h_buf, self.q_buf, self.k_buf
        slots = self.cache.begin_step(B) if self.compressed else None
        delta, summed = None, False
        for li, (qkv, o, gu, d) in enumerate(self.blocks):
            if self.pre_qkv and (delta is None or summed or self.world == 1):
                y, x = self._prenorm_linear(qkv, x, delta)
            else:
                self._add_norm(x, delta, h, summed)
                y = qkv(h)
            if self.compressed:
                layer = self.cache.layers[li]               # norm + rope of q and k and the append of k, v: one launch
                kv_ext().rope_append(y, self.head_norm_w, self.head_norm_w, self.cos, self.sin, self.pos_buf, qb,
                                     self.hq, self.hkv, c.eps, slots, layer.pages, layer.pool, layer.pcnt)
                att = layer.attention(qb, self.cache.bt32[:B], self.cache.lens[:B], scale, self.splits, None, 4)
            else:
                E.qk_norm_rope(y, self.head_norm_w, self.head_norm_w, self.cos, self.sin, self.pos_buf, qb, kb, c.eps)
                v = y[:, (self.hq + self.hkv) * D:].view(B, self.hkv, D)
                att = _flash()(qb.view(B, 1, self.hq, D), self.kc[li], self.vc[li], k=kb.view(B, 1, self.hkv, D),
                               v=v.unsqueeze(1), cache_seqlens=self.lens, softmax_scale=scale)
            delta, summed = self._row_parallel(o, att.reshape(B, self.hq * D))
            if self.pre_gu and (summed or self.world == 1):
                act, x = self._prenorm_linear(gu, x, delta, self.fused_act)
                if not self.fused_act:
                    y2 = act
                    act = torch.empty(B, y2.shape[1] // 2, dtype=torch.bfloat16, device=self.dev)
                    E.silu_mul(y2, act)
                delta, summed = self._row_parallel(d, act)
                continue
            self._add_norm(x, delta, h, summed)
            if c.experts:
                router, te = gu
                # softmax, top-k and renormalisation in one launch; with few pairs under expert parallelism the router
                # also maps the ids to this rank's experts (foreign pairs: weight 0), which the experts then run as is
                from .experts import SLOT_MAX
                logits = Fn.linear(h, router)
                if self.world > 1 and B * c.top_k <= SLOT_MAX:
                    ids, w = E.moe_route(logits, c.top_k, True, self.emap)
                    delta, summed = te(h, ids, w, None), False
                else:
                    ids, w = E.moe_route(logits, c.top_k, True, None)
                    delta, summed = te(h, ids, w, self.emap if self.world > 1 else None), False
                continue                                     # (the all-reduce over ranks happens in the next _add_norm)
            if self.fused_act:
                act = gu.swiglu(h)
            else:
                y = gu(h)
                act = torch.empty(B, y.shape[1] // 2, dtype=torch.bfloat16, device=self.dev)
                E.silu_mul(y, act)
            delta, summed = self._row_parallel(d, act)
        if self.pre_head and (summed or self.world == 1):
            logits, x = self._prenorm_linear(self.lm_head, x, delta)
        else:
            self._add_norm(x, delta, h, summed)
            logits = self.lm_head(h)
        if self.world > 1:
            parts = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(parts, logits, group=self.group)
            logits = torch.cat(parts, 1)
        if self.compressed:
            self.cache.end_step()
        else:
            self.lens += 1
        self.pos_buf += 1
        return logits

    def capture(self):
        from .kvcache import decode_splits
        self.splits = decode_splits(self.B, self.hkv, (self.max_len + 15) // 16) if self.compressed else 1
        self.next_tok = torch.zeros(self.B, dtype=torch.long, device=self.dev)
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))      # weights and buffers were written on that stream
        with torch.cuda.stream(side):
            for _ in range(2):                                   # warm-up steps (also sizes every workspace)
                self.next_tok.copy_(self._step().argmax(-1))
        side.synchronize()
        self.reset()
        torch.cuda.synchronize(self.dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):
            logits = self._step()
            self.next_tok.copy_(logits.argmax(-1))
        self.logits = logits
        self.reset()
        torch.cuda.synchronize(self.dev)
        self._check_status("capture")

    def _check_status(self, where):
        """a kernel that gave up on a bounded wait (a peer that never arrived) leaves its output unwritten: fail loudly"""
        from .ops import device_status
        with torch.cuda.device(self.dev):
            code = device_status()
        if code != 0:
            raise RuntimeError(f"TreeDecoder.{where}: a kernel gave up on a bounded wait (device status {code}); the "
                               "results of this call are invalid")

    def reset(self):
        self.pos_buf.zero_()
        if self.compressed:
            self.cache.reset()
        else:
            self.lens.zero_()

    def run(self, prompt, n_new, collect=None, margins=None):
        """prompt [B, P] token ids (teacher-forced one step at a time), then n_new greedy tokens -> [B, n_new].
        collect (optional list): receives the model's prediction after every prompt step (teacher-forced top-1).
        margins (optional list): receives, per generated token, the top-2 logit margin of sequence 0 that chose it."""
        start = int(self.pos_buf.item())
        if start + prompt.shape[1] + n_new > self.max_len:       # beyond it the page lookup would leave the block table
            raise ValueError(f"TreeDecoder.run: {prompt.shape[1]} prompt + {n_new} new tokens from position {start} "
                             f"exceed the cache capacity of {self.max_len} tokens")
        out = []
        for t in range(prompt.shape[1]):
            self.tokens.copy_(prompt[:, t])
            self.graph.replay()
            if collect is not None:
                collect.append(self.next_tok.clone())
        for _ in range(n_new):
            if margins is not None:
                top2 = self.logits[0].float().topk(2).values
                margins.append(top2[0] - top2[1])
            self.tokens.copy_(self.next_tok)
            out.append(self.next_tok.clone())
            self.graph.replay()
        res = torch.stack(out, 1) if out else torch.empty(self.B, 0, dtype=torch.long, device=self.dev)
        if self.world > 1:
            self._check_status("run")
        return res
