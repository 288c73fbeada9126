"""fp64 restatement of one Qwen3-architecture decode step as the decode runner of this repository wires it
(statetree_b200/decoder.py; the reference's own harness is statetree/bench.py:74-133, which leaves the model to
Hugging Face): RMSNorm, fused q/k/v projection, per-head q/k RMSNorm + interleaved-pair rotary embedding, grouped-query
attention over everything stored so far, output projection, SwiGLU MLP, untied lm_head.  Every product and reduction
is exact fp64; values are rounded to BF16 exactly where the GPU path stores BF16 (each kernel's output), so the two
differ only by fp32-versus-fp64 summation inside a kernel.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).
"""
import numpy as np

from . import bf16_bits_to_f32, f32_to_bf16_bits


def bf16(x):
    """round to BF16 (through fp32, nearest even), back in fp64"""
    return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x, dtype=np.float64).astype(np.float32))).astype(np.float64)


def rms(x, w, eps):
    """the two-rounding RMSNorm of the glue kernels: normalised value rounded, then scaled by the weight and rounded"""
    r = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return bf16(bf16(x * r) * w)


class OracleDecoder:
    """weights: dict of fp64 arrays (exactly the BF16 values the trees decode to):
    embed [V, H], lm_head [V, H], layers: list of dict(q [hq*128, H], k, v [hkv*128, H], o [H, hq*128], gate, up [I, H],
    down [H, I]); cos / sin [max_len, 64] (the runner's fp32 tables)"""

    def __init__(self, weights, heads, kv_heads, eps, cos, sin):
        self.w, self.hq, self.hkv, self.eps = weights, heads, kv_heads, eps
        self.cos, self.sin = np.asarray(cos, np.float64), np.asarray(sin, np.float64)
        self.K = [[] for _ in weights["layers"]]          # per layer: list over positions of [B, hkv, 128]
        self.V = [[] for _ in weights["layers"]]
        self.pos = 0
        self.x = None

    def _rope(self, heads):
        """heads [B, n, 128]: per-head RMSNorm (weight 1) then rotation of the pairs (2i, 2i + 1) by position self.pos"""
        n = rms(heads, 1.0, self.eps)
        a, b = n[..., 0::2], n[..., 1::2]
        c, s = self.cos[self.pos], self.sin[self.pos]
        out = np.empty_like(n)
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = a * s + b * c
        return bf16(out)

    def step(self, tokens):
        """tokens [B] -> logits [B, V] (BF16 values in fp64)"""
        W, hq, hkv = self.w, self.hq, self.hkv
        x = W["embed"][tokens]
        delta = None
        B = x.shape[0]
        G = hq // hkv
        for li, L in enumerate(W["layers"]):
            if delta is not None:
                x = bf16(x + delta)
            h = rms(x, 1.0, self.eps)
            q = bf16(h @ L["q"].T).reshape(B, hq, 128)
            k = bf16(h @ L["k"].T).reshape(B, hkv, 128)
            v = bf16(h @ L["v"].T).reshape(B, hkv, 128)
            q, k = self._rope(q), self._rope(k)
            self.K[li].append(k)
            self.V[li].append(v)
            Kc, Vc = np.stack(self.K[li], 1), np.stack(self.V[li], 1)        # [B, T, hkv, 128]
            att = np.empty((B, hq, 128))
            for hh in range(hq):
                s = np.einsum("bd,btd->bt", q[:, hh], Kc[:, :, hh // G]) / np.sqrt(128.0)
                p = np.exp(s - s.max(-1, keepdims=True))
                p /= p.sum(-1, keepdims=True)
                att[:, hh] = np.einsum("bt,btd->bd", p, Vc[:, :, hh // G])
            att = bf16(att).reshape(B, hq * 128)
            delta = bf16(att @ L["o"].T)
            x = bf16(x + delta)
            h = rms(x, 1.0, self.eps)
            g, u = bf16(h @ L["gate"].T), bf16(h @ L["up"].T)
            act = bf16(bf16(g / (1.0 + np.exp(-g))) * u)
            delta = bf16(act @ L["down"].T)
        x = bf16(x + delta)
        h = rms(x, 1.0, self.eps)
        self.pos += 1
        return bf16(h @ W["lm_head"].T)
