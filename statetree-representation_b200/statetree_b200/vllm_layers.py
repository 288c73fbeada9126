"""The layer methods of the reference's vLLM integration (statetree/_vllm.py, written against vLLM 0.32), without
vLLM: what happens to a layer's weights after loading and how the layer is applied.

vLLM gives every linear, embedding and fused-MoE layer a "quant method" object with two hooks,
`process_weights_after_loading(layer)` and `apply(layer, x, ...)`.  The reference installs methods that let vLLM load
the BF16 weights as usual (tensor-parallel shards, merged q/k/v and gate/up), then replace them by state trees and run
the tree kernels in `apply` (statetree/_vllm.py:218-245 linear, 266-315 embeddings / lm_head, 339-477 experts).  The
classes below are those methods, duck-typed: they touch only the attributes vLLM's layers have (`weight`,
`w13_weight` / `w2_weight`), so they can be tested on plain objects; `install()` says whether this vLLM can take them.
"""
import os

import torch
import torch.nn.functional as Fn

from .experts import TreeExperts
from .linear import EscapeHeavy, TreeEmbedding, TreeLinear
from .model import MAX_ESCAPE_FRACTION

PLAN_BATCHES = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)     # batch buckets workspaces are sized for before graph capture


def min_params():
    """linear layers with fewer weights stay BF16 (STATETREE_MIN_PARAMS, default 2^21; 0 converts every layer): below
    that a tree kernel's fixed cost exceeds the time it takes to read the matrix (statetree/_vllm.py:168-173)"""
    return int(os.environ.get("STATETREE_MIN_PARAMS", str(1 << 21)))


def supported(w):
    return w.dim() == 2 and w.dtype == torch.bfloat16 and w.is_cuda and w.shape[0] % 16 == 0 and w.shape[1] % 64 == 0


def _empty_like_param(w):
    return torch.nn.Parameter(torch.empty(0, dtype=w.dtype, device=w.device), requires_grad=False)


def _attach(layer, tree_module):
    """layer.statetree = tree_module, as a registered submodule where the layer is a module (its buffers then travel
    with the layer's state dict and device moves)"""
    if isinstance(layer, torch.nn.Module):
        layer.__dict__.pop("statetree", None)
        layer.register_module("statetree", tree_module)
    else:
        layer.statetree = tree_module


def _warm(layer, batches):
    """side tables and workspaces for every batch bucket now, so nothing is allocated or synchronised inside a later
    CUDA-graph capture"""
    layer.tables()
    with torch.no_grad():
        for b in batches:
            layer(torch.zeros(b, layer.in_features, dtype=torch.bfloat16, device=layer.tree.device))


class StateTreeLinearMethod:
    """After loading, the layer's BF16 `weight` [out, in] becomes a TreeLinear registered as `layer.statetree` and the
    BF16 tensor is released; `apply` runs it.  Matrices the format cannot hold, tiny ones and escape-heavy ones stay
    BF16 (`layer.statetree = None`) and `apply` is the plain product."""

    def __init__(self, prefix="", verify=None, batches=PLAN_BATCHES):
        self.prefix = prefix
        self.verify = (os.environ.get("STATETREE_VLLM_VERIFY", "1") != "0") if verify is None else bool(verify)
        self.batches = tuple(batches)

    def process_weights_after_loading(self, layer):
        w = layer.weight.data
        layer.statetree = None
        if not supported(w) or w.numel() < min_params():
            return
        try:
            tl = TreeLinear.from_weight(w, None, verify=self.verify, max_escape_fraction=MAX_ESCAPE_FRACTION)
        except EscapeHeavy:
            return                                           # its tree would be larger and slower than BF16
        layer.weight = _empty_like_param(layer.weight)
        _attach(layer, tl)
        _warm(tl, self.batches)

    def apply(self, layer, x, bias=None):
        tl = getattr(layer, "statetree", None)
        if tl is None:
            return Fn.linear(x, layer.weight, bias)
        y = tl(x)
        return y if bias is None else y + bias


class StateTreeEmbeddingMethod(StateTreeLinearMethod):
    """The same for a vocabulary-parallel embedding table and the output head: `embedding` looks rows up from the tree
    (exact BF16 rows), `apply` is the head's product.  `lm_head=True` converts whatever its size."""

    def __init__(self, prefix="", lm_head=False, verify=None, batches=PLAN_BATCHES):
        super().__init__(prefix, verify, batches)
        self.lm_head = lm_head

    def process_weights_after_loading(self, layer):
        w = layer.weight.data
        layer.statetree = None
        if not supported(w):
            return
        try:
            tl = TreeLinear.from_weight(w, None, verify=self.verify, max_escape_fraction=MAX_ESCAPE_FRACTION)
        except EscapeHeavy:
            return
        layer.weight = _empty_like_param(layer.weight)
        tl.allow_dec = False                                 # a vocabulary-sized table never gets a dense scratch copy
        _attach(layer, tl)
        tl.tables()
        if self.lm_head:
            _warm(tl, self.batches)

    def embedding(self, layer, input_):
        tl = getattr(layer, "statetree", None)
        if tl is None:
            return Fn.embedding(input_, layer.weight)
        return TreeEmbedding(tl.out_features, tl.in_features, source=tl)(input_)


class StateTreeMoEMethod:
    """Fused-MoE layers: vLLM loads `w13_weight` [E, 2I, H] (gate rows first) and `w2_weight` [E, H, I] for this rank's
    experts; after loading they become a TreeExperts (`layer.statetree`).  `apply(layer, x, topk_weights, topk_ids)`
    takes the router's choice; ids outside [0, E) (expert parallelism: another rank's experts, mapped to -1 or >= E by
    the caller's expert map) contribute nothing."""

    def __init__(self, prefix="", verify=None):
        self.prefix = prefix
        self.verify = (os.environ.get("STATETREE_VLLM_VERIFY", "1") != "0") if verify is None else bool(verify)

    def process_weights_after_loading(self, layer):
        w13, w2 = layer.w13_weight.data, layer.w2_weight.data
        layer.statetree = None
        ok = (w13.dim() == 3 and w2.dim() == 3 and w13.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16 and w13.is_cuda
              and w13.shape[1] % 32 == 0 and w13.shape[2] % 64 == 0 and w2.shape[1] % 16 == 0 and w2.shape[2] % 64 == 0
              and w13.shape[1] == 2 * w2.shape[2] and w13.shape[2] == w2.shape[1])
        if not ok:
            return
        te = TreeExperts.from_weights(w13, w2, verify=self.verify)
        te.sentinels = True
        layer.w13_weight, layer.w2_weight = _empty_like_param(layer.w13_weight), _empty_like_param(layer.w2_weight)
        _attach(layer, te)
        te.tables()

    def apply(self, layer, x, topk_weights, topk_ids):
        te = getattr(layer, "statetree", None)
        if te is None:
            raise RuntimeError("StateTreeMoEMethod.apply: the layer kept its BF16 experts; use the framework's own method")
        ids = topk_ids
        if ids.dtype not in (torch.int32, torch.int64):
            ids = ids.to(torch.int64)
        ids = torch.where(ids < 0, torch.full_like(ids, te.num_experts), ids)     # -1 (unmapped) -> "not mine"
        return te(x, ids, topk_weights)


def install():
    """Hook the methods into vLLM (statetree/_vllm.py:16-27 `install`, 144-152, 254-263, 485-501).  That needs the layer
    classes of vLLM 0.32 (`LinearBase.quant_method`, `UnquantizedEmbeddingMethod`, the fused-MoE method factory); this
    package does not patch other versions.  Returns (installed, reason)."""
    try:
        import vllm
    except ImportError:
        return False, "vLLM is not installed"
    version = getattr(vllm, "__version__", "0")
    return False, (f"vLLM {version}: the layer methods (StateTreeLinearMethod, StateTreeEmbeddingMethod, StateTreeMoEMethod) "
                   "are built and tested on their own; hooking them in is written for vLLM 0.32 only (vLLM 0.32 absent)")
