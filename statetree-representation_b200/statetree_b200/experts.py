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


def moe_gemv(tables, x, ids, M, xdiv, cfg=None):
    """y[s] = W[ids[s]] x[s // xdiv] for every slot s; ids int32 / int64, clamped to [0, E) in the kernel.  cfg (the
    reference's kernel configuration, statetree/experts.py:52) is accepted and ignored: the grid is chosen in the
    library."""
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


def moe_group_gemv(tables, x, aligned, S, M, xdiv, NT=1, E=None, cfg=None, zero=False):
    """y[s] = W[expert of s] x[s // xdiv], slots grouped by expert: aligned = moe_align(ids, E, 8).  Rows of blocks
    whose expert id is negative or >= the number of tables (another rank's expert) are left untouched (zero=True:
    they read as zeros).  NT / E / cfg keep the reference's argument order (statetree/experts.py:152): blocks are
    always 8 slots here (NT = 1; larger groups go to moe_group_gemm), E and cfg are not needed."""
    if NT != 1:
        raise ValueError("moe_group_gemv: blocks of 8 slots only (NT = 1); use moe_group_gemm for blocks of 64 / 128")
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


def moe_gemv_w(tables, x, ids, M, xdiv, nbps=None):
    """moe_gemv under the name the reference gives its small-K kernel (statetree/experts.py:270-279): one GEMV kernel
    serves every K here, so this is the same call; nbps (the reference's blocks per SM) has no meaning and is ignored"""
    return moe_gemv(tables, x, ids, M, xdiv)


def moe_group_gemv_w(tables, x, aligned, S, M, xdiv, nbps=None):
    """moe_group_gemv under the reference's small-K name (statetree/experts.py:282-290); nbps is ignored"""
    return moe_group_gemv(tables, x, aligned, S, M, xdiv)


def moe_fused_decode(t13, t2, x, ids, w, I):
    """out[t] = sum_j w[t, j] W2[e] (silu(W13gate[e] x[t]) * W13up[e] x[t]), e = ids[t k + j]: the routed-expert block
    of a decode step (statetree/experts.py:231-249).  t13 / t2: pointer tables of the [2I, H] gate-up (gate rows first)
    and [H, I] down trees, x [T, H] BF16, ids [T k] int32 / int64, w [T, k] routing weights.  The reference has one
    launch for it (off by default there); here it is the four launches TreeExperts uses: slot GEMV, silu * up, slot
    GEMV, weighted sum.  Deterministic."""
    x = _aligned(x)
    T, H = x.shape
    K = w.shape[-1]
    gu = moe_gemv(t13, x, ids, 2 * I, K)
    y = moe_gemv(t2, silu_mul(gu), ids, H, 1)
    return moe_wsum(y, w.reshape(T, K))


def silu_mul(gu):
    """act = silu(gate) * up for gu [S, 2I] = [gate | up] (silu in fp32, rounded to BF16, then the product)"""
    gu = _aligned(gu)
    act = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=torch.bfloat16, device=gu.device)
    ext().silu_mul(gu, act)
    return act


UP_NAMES = ("gate_up_proj", "up_proj")


def expert_layout(mod):
    """What a Transformers experts module (3-D `gate_up_proj` / `up_proj` and `down_proj` parameters, with the layout
    flags its `use_experts_implementation` decorator sets) looks like: (name of the up projection, stored transposed,
    has biases), or None for anything else.  A module without `is_transposed` is left alone, its layout cannot be known;
    one without `has_gate` is accepted only when the up projection is called gate_up_proj
    (reference: statetree/experts.py:301-320)."""
    if isinstance(mod, TreeExperts) or not hasattr(mod, "is_transposed"):
        return None
    params = mod._parameters
    up = None
    for name in UP_NAMES:
        t = params.get(name)
        if isinstance(t, torch.Tensor) and t.dim() == 3:
            up = name
            break
    down = params.get("down_proj")
    if up is None or not isinstance(down, torch.Tensor) or down.dim() != 3 or down.shape[0] != params[up].shape[0]:
        return None
    if up != "gate_up_proj" and not hasattr(mod, "has_gate"):
        return None
    biased = bool(getattr(mod, "has_bias", False))
    if biased and not all(isinstance(params.get(n + "_bias"), torch.Tensor) for n in (up, "down_proj")):
        return None
    return up, bool(mod.is_transposed), biased


def _expert_shape(P, transposed):
    """(out, in) of one expert's matrix inside the 3-D parameter P"""
    return (int(P.shape[2]), int(P.shape[1])) if transposed else (int(P.shape[1]), int(P.shape[2]))


def experts_eligible(mod, layout):
    """BF16 tensors on a real device whose per-expert matrices fit the format (out % 16 == 0, in % 64 == 0)
    (reference: statetree/experts.py:328-334)"""
    up, transposed, _ = layout
    U, D = mod._parameters[up], mod._parameters["down_proj"]
    if any(t.dtype != torch.bfloat16 or t.device.type == "meta" for t in (U, D)):
        return False
    return all(o % 16 == 0 and i % 64 == 0 for o, i in (_expert_shape(U, transposed), _expert_shape(D, transposed)))


class TreeExperts(nn.Module):
    """Routed experts with tree-stored weights; a drop-in for a Transformers 5 experts module.

    forward(hidden_states [T, H], top_k_index [T, k], top_k_weights [T, k]) -> [T, H].  The experts' matrices are the
    TreeLinear layers '<up name>.<e>' (gate_up_proj: [2I, H], gate rows first; or up_proj) and 'down_proj.<e>' ([H, I]),
    so the state dict carries the reference's keys (reference: statetree/experts.py:337-372).  SwiGLU experts without
    biases (the usual case) run on the fused kernels; other gatings, biases or a post-expert norm go expert by expert
    through the source module's own activation."""

    def __init__(self, w13, w2, up_name="gate_up_proj", source=None, has_bias=False):
        super().__init__()
        self.up_name, self.has_bias = up_name, bool(has_bias)
        self.src_class, self._gate_fn, self.config = None, None, None
        self.has_gate, self.has_post_expert_norm = up_name == "gate_up_proj", False
        if source is not None:
            # keep what the source module's forward needs: its flags and scalars, its activation / norm submodules, its
            # class's gating function
            for key, val in vars(source).items():
                if not key.startswith("_") and key != "training" and isinstance(val, (bool, int, float, str)):
                    setattr(self, key, val)
            self.config = getattr(source, "config", None)
            for key, sub in source._modules.items():
                if sub is not None:
                    self.add_module(key, sub)
            self._gate_fn = getattr(type(source), "_apply_gate", None)
            self.src_class = f"{type(source).__module__}.{type(source).__qualname__}"
            self.has_gate = bool(getattr(source, "has_gate", up_name == "gate_up_proj"))
            self.has_post_expert_norm = bool(getattr(source, "has_post_expert_norm", False))
            self.up_name, self.has_bias = up_name, bool(has_bias)
        self.add_module(up_name, nn.ModuleList(w13))
        self.down_proj = nn.ModuleList(w2)
        self.num_experts = len(self.down_proj)
        up0 = self.w13[0]
        self.hidden = up0.in_features
        self.inter = up0.out_features // 2 if self.has_gate else up0.out_features
        self._tabs = None
        self._maps = None
        self.sentinels = source is not None                 # callers of the Transformers interface may pass ids >= E

    @property
    def w13(self):
        return getattr(self, self.up_name)

    @property
    def w2(self):
        return self.down_proj

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        self._tabs = self._maps = None                      # the trees may have moved
        return out

    @classmethod
    @torch.no_grad()
    def from_weights(cls, gate_up, down, verify=True):
        """gate_up [E, 2I, H], down [E, H, I] bf16"""
        return cls([TreeLinear.from_weight(gate_up[e], verify=verify) for e in range(gate_up.shape[0])],
                   [TreeLinear.from_weight(down[e], verify=verify) for e in range(down.shape[0])])

    @classmethod
    @torch.no_grad()
    def from_experts(cls, source, verify=True):
        """Encode every expert of a Transformers experts module (see expert_layout).  Each 3-D BF16 tensor is dropped
        from the source module as soon as its trees exist, so the peak is one tensor plus its trees."""
        layout = expert_layout(source)
        if layout is None or not experts_eligible(source, layout):
            raise ValueError("TreeExperts.from_experts: not a BF16 experts module this format can hold")
        up, transposed, biased = layout
        params = source._parameters
        lists = {}
        for name in (up, "down_proj"):
            P = params[name]
            bias = params.get(name + "_bias") if biased else None
            mods = []
            for e in range(int(P.shape[0])):
                W = P[e].t().contiguous() if transposed else P[e]
                mods.append(TreeLinear.from_weight(W, None if bias is None else bias[e], verify=verify))
            lists[name] = mods
            del P, bias
            params.pop(name)
            params.pop(name + "_bias", None)
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
        return cls(lists[up], lists["down_proj"], up_name=up, source=source, has_bias=biased)

    def spec(self):
        """what load_pretrained needs, beside the model's config, to build this module empty"""
        u, d = self.w13[0], self.w2[0]
        return dict(up=self.up_name, num_experts=self.num_experts, up_shape=[u.out_features, u.in_features],
                    down_shape=[d.out_features, d.in_features], bias=self.has_bias, source=self.src_class)

    @classmethod
    def skeleton(cls, source, spec):
        """an empty (meta) TreeExperts in the place of `source`, to be filled by load_state_dict"""
        (uo, ui), (do, di) = spec["up_shape"], spec["down_shape"]
        n, biased = int(spec["num_experts"]), bool(spec["bias"])
        return cls([TreeLinear(ui, uo, bias=biased, device="meta") for _ in range(n)],
                   [TreeLinear(di, do, bias=biased, device="meta") for _ in range(n)],
                   up_name=spec["up"], source=source, has_bias=biased)

    def storage_bytes(self):
        return sum(m.storage_bytes() for m in self.modules() if isinstance(m, TreeLinear))

    def extra_repr(self):
        up, down = self.w13[0], self.down_proj[0]
        weights = sum(m.in_features * m.out_features for m in self.modules() if isinstance(m, TreeLinear))
        return (f"{self.num_experts} experts as state trees: {self.up_name} {up.out_features}x{up.in_features}, down_proj "
                f"{down.out_features}x{down.in_features}, gate={self.has_gate}, bias={self.has_bias}, "
                f"{8 * self.storage_bytes() / max(1, weights):.2f} bits per weight")

    def _fast_ok(self):
        """the fused kernels compute silu(gate) * up of a [2I, H] gate_up_proj without biases: the default gating"""
        act = getattr(self, "act_fn", None)
        plain_gate = self._gate_fn is None or getattr(self._gate_fn, "__name__", "") == "_default_apply_gate"
        silu = act is None or isinstance(act, nn.SiLU) or "SiLU" in type(act).__name__
        u, d = self.w13[0], self.w2[0]
        return (self.has_gate and not self.has_bias and not self.has_post_expert_norm and plain_gate and silu
                and self.up_name == "gate_up_proj" and u.out_features == 2 * d.in_features
                and u.in_features == d.out_features)

    def _gated(self, h):
        if self._gate_fn is not None:
            return self._gate_fn(self, h)
        gate, up = h.chunk(2, dim=-1)
        act = getattr(self, "act_fn", None)
        return (act(gate) if act is not None else torch.nn.functional.silu(gate)) * up

    def _expert_by_expert(self, x, ids, w, T, K):
        """every pair through its expert's TreeLinear layers, experts in turn (biases live in the layers); ids >= E
        (another rank's experts) contribute nothing"""
        E = self.num_experts
        order = torch.sort(ids.long()).indices
        sorted_ids = ids.long()[order]
        rows = x[order // K]
        counts = torch.bincount(sorted_ids.clamp(max=E), minlength=E + 1)[:E].tolist()
        out = x.new_zeros(rows.shape[0], self.w2[0].out_features)
        at = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            h = self.w13[e](rows[at:at + n])
            h = self._gated(h) if self.has_gate else self.act_fn(h)
            out[at:at + n] = self.w2[e](h)
            at += n
        if self.has_post_expert_norm:
            out = self.post_expert_norm(out)
        out = out * w.reshape(-1)[order].to(out.dtype).unsqueeze(-1)
        back = torch.empty_like(order)
        back[order] = torch.arange(order.numel(), device=order.device)
        return out[back].view(T, K, -1).sum(1).to(x.dtype)

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

    def forward(self, hidden_states, top_k_index, top_k_weights, expert_map=None):
        """The call of a Transformers experts module (statetree/experts.py: TreeExperts.forward).  expert_map (optional
        int32 [E_global]): global expert id -> local id or -1 (expert parallelism); pairs of other ranks' experts
        contribute zero."""
        x, topk_ids, topk_w = hidden_states, top_k_index, top_k_weights
        T, K = topk_ids.shape
        S = T * K
        if S == 0:
            return x.new_zeros(T, self.w2[0].out_features)
        if not (self._fast_ok() and x.is_cuda):
            ids = topk_ids.reshape(-1)
            if expert_map is not None:
                local = expert_map[ids.long()]
                ids = torch.where(local >= 0, local, torch.full_like(local, self.num_experts))
            return self._expert_by_expert(x, ids, topk_w, T, K)
        asked = x.dtype
        if asked != torch.bfloat16:
            x = x.to(torch.bfloat16)
        x = _aligned(x)
        if self.sentinels and expert_map is None:
            # ids >= E mark pairs of another rank's experts (the convention of expert-parallel callers): weight 0
            valid = topk_ids < self.num_experts
            topk_w = torch.where(valid, topk_w, torch.zeros_like(topk_w))
            topk_ids = topk_ids.clamp(max=self.num_experts - 1)
        if topk_ids.dtype not in (torch.int32, torch.int64):
            topk_ids = topk_ids.to(torch.int64)
        out = self._fast(x, topk_ids.contiguous(), topk_w, expert_map, T, K, S)
        return out if asked == torch.bfloat16 else out.to(asked)

    def _fast(self, x, topk_ids, topk_w, expert_map, T, K, S):
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
