"""Mixture-of-experts products over tree-stored expert matrices: the wrappers of the reference's statetree/experts.py
(moe_gemv 52-66, expert_tables 74-85, moe_align 123-141, moe_group_gemv 152-162, moe_wsum 291-298) and a TreeExperts
block (reference 337-519) over the sm_100a kernels.  One kernel serves both slot layouts; there is no per-size ladder
beyond "few pairs: one problem per (token, expert) slot; many pairs: slots grouped by expert, each expert's records
read once per block of 8 slots".
"""

import torch
import torch.nn as nn

from .linear import TreeLinear, _state
from .ops import ext

SLOT_MAX = 32                       # (token, expert) pairs up to which the ungrouped kernel runs
GEMM_PAIRS_PER_EXPERT = 8           # average pairs per expert from which the grouped tcgen05 GEMM takes over: the
#                                     grouped GEMV re-reads an expert's records for every 8 of its pairs, the GEMM
#                                     reads them once per 64 (128 from 64 pairs per expert on)


def _aligned(x):
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    if not x.is_contiguous() or x.data_ptr() % 16:
        x = x.clone(memory_format=torch.contiguous_format)
    return x


class PtrTables(tuple):
    """(TP, EOP, EBP, ELP) int64 device-address tables, one entry per expert; .keep pins the tensors they point into"""


def expert_tables(mods):
    """address tables of a list of same-shape per-expert TreeLinear layers (side tables are built now)"""
    dev = mods[0].tree.device
    cols = ([], [], [], [])
    keep = []
    for m in mods:
        eo, el, eb = m.tables()
        for lst, t in zip(cols, (m.tree, eo, eb, el)):
            lst.append(t.data_ptr())
        keep += [m.tree, eo, eb, el]
    t = PtrTables(torch.tensor(v, dtype=torch.int64, device=dev) for v in cols)
    t.keep = keep
    return t


def moe_gemv(tables, x, ids, M, xdiv):
    """y[s] = W[ids[s]] x[s // xdiv] for every slot s; ids int32 / int64, clamped to [0, E) in the kernel"""
    x = _aligned(x)
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    ids = ids.reshape(-1).contiguous()
    S, N = ids.numel(), x.shape[1]
    y = torch.empty(S, M, dtype=torch.bfloat16, device=x.device)
    if S == 0:
        return y
    E = ext()
    st = _state(x.device)
    ws = st.get_ws(E.moe_gemv_workspace_bytes(S, M, N))
    E.mvx(*tables, x, ids, y, ws, st.get_cnt(S * (M // 16)), xdiv)
    return y


def moe_align(ids, E, bs=8, used_bins=None):
    """Pairs grouped by expert in blocks of bs (the moe_align_block_size layout), with torch ops and no host sync:
    (sorted_ids int32 [nblk * bs], padded with S; bexp int32 [nblk]; npost int32 [1] = entries of the first used_bins
    experts, default all E: the grouped kernel does not visit blocks beyond it)."""
    ids = ids.reshape(-1)
    S, dev = ids.numel(), ids.device
    nblk = S // bs + min(S, E) + 1
    if (ids.is_cuda and 1 <= S <= (1 << 20) and E <= 1024
            and ids.dtype in (torch.int64, torch.int32)):
        # one CTA of the kernel library does the whole grouping (the torch formulation below is ~20 small launches)
        sorted_ids = torch.empty(nblk * bs, dtype=torch.int32, device=dev)
        bexp = torch.empty(nblk, dtype=torch.int32, device=dev)
        npost = torch.empty(1, dtype=torch.int32, device=dev)
        ext().moe_align(ids.contiguous(), E, E if used_bins is None else used_bins, sorted_ids, bexp, npost, bs)
        return sorted_ids, bexp, npost
    return _moe_align_torch(ids, E, bs, used_bins)


def _moe_align_torch(ids, E, bs=8, used_bins=None):
    """the same layout with torch ops (CPU tensors, other block sizes, very long calls); the check for the kernel"""
    ids = ids.reshape(-1).to(torch.int64)
    S, dev = ids.numel(), ids.device
    nblk = S // bs + min(S, E) + 1
    per = torch.zeros(E, dtype=torch.int64, device=dev).scatter_add_(0, ids.clamp(0, E - 1), torch.ones_like(ids))   # no sync
    room = (per + bs - 1) // bs * bs                     # slots reserved per expert
    end = room.cumsum(0)
    begin = end - room
    by_expert = torch.argsort(ids, stable=True)          # pair indices, expert-major, original order inside
    e_sorted = ids[by_expert]
    rank = torch.arange(S, device=dev) - (per.cumsum(0) - per)[e_sorted]
    sorted_ids = torch.full((nblk * bs,), S, dtype=torch.int32, device=dev)
    sorted_ids[begin[e_sorted] + rank] = by_expert.to(torch.int32)
    blk_start = torch.arange(nblk, device=dev) * bs
    bexp = torch.searchsorted(end, blk_start, right=True).clamp(max=E - 1).to(torch.int32)
    nb = E if used_bins is None else used_bins
    return sorted_ids, bexp, end[nb - 1:nb].to(torch.int32)


def moe_group_gemv(tables, x, aligned, S, M, xdiv, zero=False):
    """y[s] = W[expert of s] x[s // xdiv], slots grouped by expert: aligned = moe_align(ids, E, 8).  Rows of blocks
    whose expert id is negative or >= the number of tables (another rank's expert) are left untouched (zero=True:
    they read as zeros)."""
    sorted_ids, bexp, npost = (t.contiguous() for t in aligned)
    x = _aligned(x)
    N = x.shape[1]
    y = (torch.zeros if zero else torch.empty)(S, M, dtype=torch.bfloat16, device=x.device)
    if S == 0:
        return y
    E = ext()
    st = _state(x.device)
    nblk = bexp.numel()
    ws = st.get_ws(E.moe_group_workspace_bytes(nblk, M, N))
    E.mvg(*tables, x, sorted_ids, bexp, npost, y, ws, st.get_cnt(nblk * (M // 16)), xdiv)
    return y


def moe_group_gemm(tables, maps, x, aligned, bs, S, M, xdiv, zero=False, yf32=None):
    """The same product through the grouped fused decode + tcgen05 GEMM: aligned = moe_align(ids, E, bs), bs = 64 or
    128; maps = ext().moe_tensor_maps(trees, M, N).  The activation rows are first gathered into block order (one
    small kernel), each CTA then multiplies one block of pairs by 128 rows of its expert's matrix."""
    sorted_ids, bexp, npost = (t.contiguous() for t in aligned)
    x = _aligned(x)
    y = (torch.zeros if zero else torch.empty)(S, M, dtype=torch.bfloat16, device=x.device)
    if S == 0:
        return y
    E = ext()
    xg = torch.empty(sorted_ids.numel(), x.shape[1], dtype=torch.bfloat16, device=x.device)
    E.moe_gather(x, sorted_ids, npost, S, xdiv, xg)
    E.gtt(maps, tables[1], tables[3], xg, sorted_ids, bexp, npost, bs, y, yf32)
    return y


def moe_wsum(y, w):
    """out[t] = sum_j w[t, j] y[t * k + j] (fp32 sum in expert order, BF16 out); w [T, k] float32 or BF16"""
    T, K = w.shape
    out = torch.empty(T, y.shape[1], dtype=torch.bfloat16, device=y.device)
    if w.dtype not in (torch.float32, torch.bfloat16):
        w = w.float()
    ext().wsum(_aligned(y), w.contiguous(), out)
    return out


def silu_mul(gu):
    """act = silu(gate) * up for gu [S, 2I] = [gate | up] (silu in fp32, rounded to BF16, then the product)"""
    gu = _aligned(gu)
    act = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=torch.bfloat16, device=gu.device)
    ext().silu_mul(gu, act)
    return act


class TreeExperts(nn.Module):
    """Routed SwiGLU experts with tree-stored weights: w13[e] [2I, H] (gate rows first) and w2[e] [H, I].

    forward(x [T, H], topk_ids [T, k], topk_w [T, k]) -> [T, H] = sum_j w[t, j] W2[e] (silu(Wg[e] x) * Wu[e] x)."""

    def __init__(self, w13, w2):
        super().__init__()
        self.w13, self.w2 = nn.ModuleList(w13), nn.ModuleList(w2)
        self.num_experts = len(w13)
        self.hidden, self.inter = w13[0].in_features, w13[0].out_features // 2
        self._tabs = None
        self._maps = None

    @classmethod
    @torch.no_grad()
    def from_weights(cls, gate_up, down, verify=True):
        """gate_up [E, 2I, H], down [E, H, I] bf16"""
        return cls([TreeLinear.from_weight(gate_up[e], verify=verify) for e in range(gate_up.shape[0])],
                   [TreeLinear.from_weight(down[e], verify=verify) for e in range(down.shape[0])])

    def tables(self):
        if self._tabs is None:
            self._tabs = (expert_tables(list(self.w13)), expert_tables(list(self.w2)))
        return self._tabs

    def tensor_maps(self):
        """weight tensor maps of the grouped tcgen05 GEMM, or None when the shapes do not fit it (rows % 128)"""
        if self._maps is None:
            if (2 * self.inter) % 128 or self.hidden % 128:
                self._maps = False
            else:
                E = ext()
                self._maps = (E.moe_tensor_maps([m.tree for m in self.w13], 2 * self.inter, self.hidden),
                              E.moe_tensor_maps([m.tree for m in self.w2], self.hidden, self.inter))
        return self._maps or None

    def record_bytes(self):
        return sum(m.record_bytes() for m in self.w13) + sum(m.record_bytes() for m in self.w2)

    def forward(self, x, topk_ids, topk_w, expert_map=None):
        """expert_map (optional int32 [E_global]): global expert id -> local id or -1 (expert parallelism); pairs of
        other ranks' experts contribute zero."""
        T, K = topk_ids.shape
        S = T * K
        t13, t2 = self.tables()
        ids = topk_ids.reshape(-1)
        w = topk_w
        if expert_map is not None:
            # expert parallel: pairs of other ranks' experts go to one extra bin whose blocks the kernel skips
            local = expert_map[ids.long()]
            w = torch.where(local.view(T, K) >= 0, topk_w, torch.zeros_like(topk_w))
            if S <= SLOT_MAX:                           # a few pairs: cheaper to compute them all (weight 0) than to group
                ids = local.clamp(min=0)
                gu = moe_gemv(t13, x, ids, 2 * self.inter, K)
                return moe_wsum(moe_gemv(t2, silu_mul(gu), ids, self.hidden, 1), w)
            ids = torch.where(local >= 0, local, torch.full_like(local, self.num_experts))
            al = moe_align(ids, self.num_experts + 1, 8, used_bins=self.num_experts)   # the last bin = other ranks' pairs
            gu = moe_group_gemv(t13, x, al, S, 2 * self.inter, K, zero=True)
            y = moe_group_gemv(t2, silu_mul(gu), al, S, self.hidden, 1, zero=True)
            return moe_wsum(y, w)
        if S <= SLOT_MAX:
            gu = moe_gemv(t13, x, ids, 2 * self.inter, K)
            y = moe_gemv(t2, silu_mul(gu), ids, self.hidden, 1)
        elif S >= GEMM_PAIRS_PER_EXPERT * self.num_experts and self.tensor_maps() is not None:
            bs = 128 if S >= 64 * self.num_experts else 64
            m13, m2 = self.tensor_maps()
            al = moe_align(ids, self.num_experts, bs)
            gu = moe_group_gemm(t13, m13, x, al, bs, S, 2 * self.inter, K)
            y = moe_group_gemm(t2, m2, silu_mul(gu), al, bs, S, self.hidden, 1)
        else:
            al = moe_align(ids, self.num_experts, 8)
            gu = moe_group_gemv(t13, x, al, S, 2 * self.inter, K)
            y = moe_group_gemv(t2, silu_mul(gu), al, S, self.hidden, 1)
        return moe_wsum(y, w)
