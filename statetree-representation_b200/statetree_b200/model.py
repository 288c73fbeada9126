"""Model-level API over the tree-stored layers: convert a model's BF16 linear layers and embedding tables in place,
prepare them for CUDA-graph capture, and save / load checkpoints in the reference's on-disk format, so that a directory
written by either implementation loads in the other (reference: statetree/model.py convert 63-216, prepare 219-241,
size_report 244-262, save_pretrained 282-310, load_pretrained 372-464).

On disk: `model.safetensors` (the state dict; tensors that share storage are written once), `statetree.json`
(format "statetree", version 3: `modules` name -> in/out features and bias of every TreeLinear, `fused` fused layer
-> [[part name, first row, rows], ...], `embeddings` name -> sizes and the tied source layer, `experts`, `aliases`
alias key -> stored key, `dtype`, `architecture`), and the model's own config files.
"""
import contextlib
import fnmatch
import gc
import json
import os
import time

import torch
import torch.nn as nn

from . import format as F
from .experts import TreeExperts, expert_layout, experts_eligible
from .linear import EscapeHeavy, TreeEmbedding, TreeLinear, TreeSlice

FORMAT_NAME = "statetree"
FORMAT_VERSION = 3                     # leaf byte = mantissa << 1 | partner's sign; version 2 files are migrated on load
WEIGHTS_NAME = "model.safetensors"
INFO_NAME = "statetree.json"
MAX_ESCAPE_FRACTION = float(os.environ.get("STATETREE_MAX_ESCAPES", "0.01"))
# sibling projections that read the same activation and are stored (and launched) as one tree
DEFAULT_FUSE = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj"),
                "in_proj_all": ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a"),
                "in_proj_qkvzba": ("in_proj_qkvz", "in_proj_ba")}


def _selected(name, patterns):
    leaf = name.rsplit(".", 1)[-1]
    return any(name == p or leaf == p or fnmatch.fnmatch(name, p) for p in patterns)


def _owner(model, dotted):
    """(module that holds the attribute, attribute name) for a dotted module path"""
    head, _, leaf = dotted.rpartition(".")
    return (model.get_submodule(head) if head else model), leaf


def _convertible(mod):
    w = getattr(mod, "weight", None)
    return (isinstance(mod, nn.Linear) and w is not None and w.dtype == torch.bfloat16 and w.device.type != "meta"
            and mod.out_features % 16 == 0 and mod.in_features % 64 == 0)


def tree_modules(model):
    """[(name, TreeLinear)] in module order"""
    return [(n, m) for n, m in model.named_modules() if isinstance(m, TreeLinear)]


@torch.no_grad()
def convert(model, include=None, exclude=(), fuse=DEFAULT_FUSE, embeddings=True, experts=True, verify=True,
            verbose=True, max_escape_fraction=None):
    """Replace, in place, every BF16 nn.Linear whose shape fits the format (out % 16 == 0, in % 64 == 0) by a
    TreeLinear, and BF16 nn.Embedding tables by TreeEmbedding.

    fuse        {fused attribute: part attributes}: siblings reading one input become one TreeLinear on their parent
                and each part a TreeSlice of its output (None: keep them apart)
    embeddings  convert embedding tables too; a table tied to the output layer shares that layer's tree
    include / exclude   module-name patterns (fnmatch, a full name, or a bare attribute name such as "lm_head")
    verify      decode every tree and compare it bit for bit with the source weights
    max_escape_fraction matrices with more escapes stay BF16 (default 1%, STATETREE_MAX_ESCAPES)
    experts     also store mixture-of-experts weights kept as 3-D parameters (Transformers 5 experts modules) as one tree
                per expert matrix: the module becomes a TreeExperts (experts held as nn.Linear modules are ordinary
                linear layers and are converted either way)"""
    t_start = time.perf_counter()
    limit = MAX_ESCAPE_FRACTION if max_escape_fraction is None else max_escape_fraction
    cfg = getattr(model, "config", None)
    head = model.get_output_embeddings() if hasattr(model, "get_output_embeddings") else None
    table = model.get_input_embeddings() if hasattr(model, "get_input_embeddings") else None
    tied = isinstance(head, nn.Linear) and isinstance(table, nn.Embedding) and head.weight is table.weight

    def chosen(name):
        if exclude and _selected(name, exclude):
            return False
        return not include or _selected(name, include)

    pending, left_out = {}, []
    for name, mod in model.named_modules():
        if isinstance(mod, nn.Linear) and chosen(name):
            if _convertible(mod):
                pending[name] = mod
            else:
                left_out.append(name)
    tally = dict(bf16=0, tree=0, linears=0, groups=0, tables=0, heavy=0, moe=0, moe_mats=0)

    # mixture-of-experts weights held as 3-D parameters: one tree per expert matrix, each BF16 tensor freed once encoded
    if experts:
        for name, mod in list(model.named_modules()):
            layout = expert_layout(mod)
            if layout is None or not chosen(name):
                continue
            if not experts_eligible(mod, layout):
                left_out.append(name)
                continue
            worst = _expert_escape_fraction(mod, layout)
            if worst > limit:
                left_out.append(f"{name} (escape-heavy: {worst:.2%})")
                tally["heavy"] += 1
                continue
            up = layout[0]
            tally["bf16"] += sum(2 * t.numel() for k, t in mod._parameters.items()
                                 if t is not None and k in (up, "down_proj", up + "_bias", "down_proj_bias"))
            te = TreeExperts.from_experts(mod, verify=verify)
            parent, attr = _owner(model, name)
            setattr(parent, attr, te)
            tally["tree"] += te.storage_bytes()
            tally["moe"] += 1
            tally["moe_mats"] += 2 * te.num_experts

    # siblings that share their input: one tree, the parts become views of its output
    for pname, parent in list(model.named_modules()):
        for fused_attr, part_attrs in (fuse or {}).items():
            paths = [f"{pname}.{a}" if pname else a for a in part_attrs]
            if hasattr(parent, fused_attr) or any(p not in pending for p in paths):
                continue
            parts = [pending[p] for p in paths]
            with_bias = [m.bias is not None for m in parts]
            if len({m.in_features for m in parts}) > 1 or (any(with_bias) and not all(with_bias)):
                continue
            stacked = torch.cat([m.weight for m in parts], 0)
            bias = torch.cat([m.bias for m in parts], 0) if all(with_bias) else None
            try:
                whole = TreeLinear.from_weight(stacked, bias, verify=verify, max_escape_fraction=limit)
            except EscapeHeavy:
                continue                                   # each part gets its own chance below
            finally:
                del stacked
            setattr(parent, fused_attr, whole)
            row = 0
            for attr, path, m in zip(part_attrs, paths, parts):
                setattr(parent, attr, TreeSlice(whole, row, m.out_features, len(parts)))
                row += m.out_features
                tally["bf16"] += 2 * m.weight.numel()
                del pending[path]
            tally["tree"] += whole.storage_bytes()
            tally["linears"] += len(parts)
            tally["groups"] += 1

    # everything else, one by one
    new_head = None
    for name in sorted(pending):
        lin = pending[name]
        try:
            tl = TreeLinear.from_linear(lin, verify=verify, max_escape_fraction=limit)
        except EscapeHeavy as why:
            left_out.append(f"{name} (escape-heavy: {why})")
            tally["heavy"] += 1
            continue
        parent, attr = _owner(model, name)
        setattr(parent, attr, tl)
        if lin is head:
            new_head = tl
        tally["bf16"] += 2 * lin.weight.numel()
        tally["tree"] += tl.storage_bytes()
        tally["linears"] += 1
    pending.clear()
    if tied and new_head is not None and cfg is not None:
        cfg.tie_word_embeddings = False                    # the tie now runs through TreeEmbedding(source=head tree)

    if embeddings:
        for name, mod in list(model.named_modules()):
            if not isinstance(mod, nn.Embedding) or not chosen(name) or mod.max_norm is not None:
                continue
            w = mod.weight
            if (w.dtype != torch.bfloat16 or w.device.type == "meta" or mod.embedding_dim % 64
                    or mod.num_embeddings % 16):
                continue
            if F.escape_count(w) > limit * w.numel():
                left_out.append(f"{name} (escape-heavy)")
                tally["heavy"] += 1
                continue
            if tied and mod is table:
                if new_head is None:
                    continue                               # the head stayed BF16: the table keeps sharing it
                emb = TreeEmbedding(mod.num_embeddings, mod.embedding_dim, source=new_head)
            else:
                emb = TreeEmbedding.from_embedding(mod, verify=verify)
                tally["tree"] += emb.table.storage_bytes()
            parent, attr = _owner(model, name)
            setattr(parent, attr, emb)
            tally["bf16"] += 2 * w.numel()
            tally["tables"] += 1
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    if verbose:
        note = f", {len(left_out)} layers left in BF16 ({tally['heavy']} escape-heavy)" if left_out else ""
        print(f"statetree_b200: {tally['linears']} linear layers ({tally['groups']} fused groups), {tally['tables']} "
              f"embedding tables in {time.perf_counter() - t_start:.1f}s: {tally['bf16'] / 2**30:.3f} GiB -> "
              f"{tally['tree'] / 2**30:.3f} GiB{note}{', all bit-exact' if verify else ''}")
    return model


def prepare(model, batch_sizes=(1,), verbose=False):
    """Everything a layer allocates lazily, done now, so that later calls (and CUDA-graph capture) allocate nothing:
    the escape side tables of every TreeLinear on a GPU and, per (device, current stream), workspaces large enough
    for every listed batch size of every shape.
    (The reference picks a kernel per batch bucket here by timing candidates; this implementation has one kernel per
    regime, so there is nothing to tune.)"""
    from .linear import GEMV_MAX, _state
    from .ops import ext
    mods = [m for _, m in tree_modules(model) if m.tree.device.type == "cuda"]
    E = ext() if mods else None
    import weakref
    for m, after in zip(mods, mods[1:] + mods[:1]):          # prefill: decode the next layer while this one multiplies
        m.__dict__["_next"] = weakref.ref(after)
    for m in mods:
        m.tables()
        st = _state(m.tree.device)
        need, M, N = 0, m.out_features, m.in_features
        for B in batch_sizes:
            if B <= min(GEMV_MAX, 32) or M % 128:
                need = max(need, E.gemv_workspace_bytes(M, N, min(B, 32)))
                st.get_cnt(M // 16)
            else:
                need = max(need, E.gemm_workspace_bytes(M, N, B))
                st.get_cnt((M // 128) * ((B + 255) // 256))
        st.get_ws(need)
        if verbose:
            print(f"statetree_b200: {M}x{N}: workspace {need} bytes for batches {tuple(batch_sizes)}")
    return model


def size_report(model):
    """storage of the tree-stored layers against BF16, and of everything else in the model"""
    layers = tree_modules(model)
    tree_bytes = sum(m.storage_bytes() for _, m in layers)
    weights = sum(m.in_features * m.out_features for _, m in layers)
    escapes = sum(m.esc_rows.numel() for _, m in layers)
    seen, total = set(), 0
    for t in list(model.parameters()) + list(model.buffers()):
        if t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    return dict(tree_layers=len(layers), tree_weights=weights, tree_bytes=tree_bytes, bf16_bytes=2 * weights,
                bits_per_weight=8 * tree_bytes / max(weights, 1), escape_fraction=escapes / max(weights, 1),
                other_bytes=total - tree_bytes, total_bytes=total)


@torch.no_grad()
def _expert_escape_fraction(mod, layout):
    """the larger of the escape fractions of the up and the down projection tensor of an experts module"""
    up, transposed, _ = layout
    worst = 0.0
    for name in (up, "down_proj"):
        P = mod._parameters[name]
        if transposed:                                     # [E, in, out]: the 64-column groups run along `in`
            n = sum(F.escape_count(P[e].t().contiguous()) for e in range(P.shape[0]))
        else:
            n = F.escape_count(P.reshape(-1, P.shape[-1]))
        worst = max(worst, n / P.numel())
    return worst


# ---------------------------------------------------------------------------------------------- checkpoints
def _describe(model):
    """the tables of statetree.json that describe module structure"""
    name_of = {id(m): n for n, m in tree_modules(model)}
    expert_specs = {n: m.spec() for n, m in model.named_modules() if isinstance(m, TreeExperts)}
    modules = {n: dict(in_features=m.in_features, out_features=m.out_features, bias=m.bias is not None)
               for n, m in tree_modules(model) if n.rsplit(".", 2)[0] not in expert_specs}   # expert trees: under `experts`
    fused, tables = {}, {}
    for n, m in model.named_modules():
        if isinstance(m, TreeSlice):
            fused.setdefault(name_of[id(m.fused)], []).append([n, m.start, m.out_features])
        elif isinstance(m, TreeEmbedding):
            tables[n] = dict(num_embeddings=m.num_embeddings, embedding_dim=m.embedding_dim,
                             source=None if m.table is not None else name_of[id(m.source)])
    return modules, fused, tables, expert_specs


def save_pretrained(model, path, tokenizer=None):
    """config files, statetree.json and model.safetensors under `path`"""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    stored, aliases, owner_of = {}, {}, {}
    for key, t in model.state_dict().items():
        ident = None
        if t.numel():
            ident = (t.device, t.untyped_storage().data_ptr(), t.storage_offset(), tuple(t.shape), tuple(t.stride()), t.dtype)
        if ident is not None and ident in owner_of:
            aliases[key] = owner_of[ident]                 # same memory as an earlier key: written once
            continue
        if ident is not None:
            owner_of[ident] = key
        stored[key] = t.detach().contiguous()
    modules, fused, tables, expert_specs = _describe(model)
    info = dict(format=FORMAT_NAME, version=FORMAT_VERSION, modules=modules, fused=fused, embeddings=tables,
                experts=expert_specs, aliases=aliases, dtype="bfloat16", architecture=type(model).__name__)
    save_file(stored, os.path.join(path, WEIGHTS_NAME), metadata={"format": "pt", FORMAT_NAME: str(FORMAT_VERSION)})
    with open(os.path.join(path, INFO_NAME), "w") as fh:
        json.dump(info, fh, indent=1)
    for extra in (getattr(model, "config", None), getattr(model, "generation_config", None), tokenizer):
        if extra is not None and hasattr(extra, "save_pretrained"):
            try:
                extra.save_pretrained(path)
            except Exception:                              # noqa: BLE001  (a generation config may refuse to validate)
                if extra is getattr(model, "config", None):
                    raise
    return path


@contextlib.contextmanager
def _parameters_on_meta():
    """while active, every parameter a module registers lands on the meta device (no memory, no initialisation);
    buffers such as rotary tables stay real"""
    original = nn.Module.register_parameter

    def on_meta(self, name, param):
        original(self, name, param)
        if param is not None:
            live = self._parameters[name]
            self._parameters[name] = type(live)(live.to("meta"), requires_grad=live.requires_grad)

    nn.Module.register_parameter = on_meta
    try:
        yield
    finally:
        nn.Module.register_parameter = original


def load_pretrained(path, device=None, device_map=None, max_memory=None, model_cls=None, **config_kwargs):
    """Rebuild a converted Hugging Face model from a directory written by save_pretrained (this implementation's or the
    reference's) without ever materialising BF16 weights.  The whole model goes to `device` (default: cuda when a GPU
    is present, else cpu); device maps over several GPUs need accelerate, which this build does not use, so
    device_map / max_memory other than None raise."""
    from safetensors.torch import load_file
    with open(os.path.join(path, INFO_NAME)) as fh:
        info = json.load(fh)
    if info.get("format") != FORMAT_NAME:
        raise ValueError(f"{path}: not a statetree checkpoint")
    if device_map not in (None, "auto") or max_memory is not None:
        raise NotImplementedError("statetree_b200.load_pretrained: one device only (pass device=...)")
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    import transformers
    from transformers import AutoConfig, AutoModelForCausalLM
    config = AutoConfig.from_pretrained(path, **config_kwargs)
    cls = model_cls or getattr(transformers, str(info.get("architecture", "")), None) or AutoModelForCausalLM
    build = getattr(cls, "from_config", None) or cls._from_config
    with _parameters_on_meta():
        try:
            model = build(config, dtype=torch.bfloat16)
        except TypeError:
            model = build(config, torch_dtype=torch.bfloat16)
    for name, spec in info.get("experts", {}).items():     # empty TreeExperts in place of the 3-D parameter modules
        parent, attr = _owner(model, name)
        setattr(parent, attr, TreeExperts.skeleton(getattr(parent, attr), spec))
    tables = info.get("embeddings", {})
    for name, e in tables.items():
        own = None if e["source"] else TreeLinear(e["embedding_dim"], e["num_embeddings"], device="meta")
        parent, attr = _owner(model, name)
        setattr(parent, attr, TreeEmbedding(e["num_embeddings"], e["embedding_dim"], table=own))
    for name, m in info["modules"].items():
        parent, attr = _owner(model, name)
        if not isinstance(getattr(parent, attr, None), TreeLinear):
            setattr(parent, attr, TreeLinear(m["in_features"], m["out_features"], bias=m["bias"], device="meta"))
    for fused_name, parts in info.get("fused", {}).items():
        whole = model.get_submodule(fused_name)
        for part_name, row, rows in parts:
            parent, attr = _owner(model, part_name)
            setattr(parent, attr, TreeSlice(whole, row, rows, len(parts)))
    for name, e in tables.items():
        if e["source"]:
            object.__setattr__(model.get_submodule(name), "source", model.get_submodule(e["source"]))
    state = load_file(os.path.join(path, WEIGHTS_NAME), device=str(device))
    if info.get("version", 2) < 3:                         # older files carry leaf format 1
        for key, t in list(state.items()):
            if key.endswith("tree") and t.dtype == torch.uint8 and t.dim() == 3 and t.shape[-1] == F.RECORD_BYTES:
                state[key] = F.leaves_v1_to_v2(t)
    for alias, src in info.get("aliases", {}).items():
        state[alias] = state[src]
    _, unexpected = model.load_state_dict(state, strict=False, assign=True)
    del state
    if getattr(config, "tie_word_embeddings", False) and hasattr(model, "tie_weights"):
        model.tie_weights()
    model.to(device)
    on_meta = [n for n, t in list(model.named_parameters()) + list(model.named_buffers()) if t.device.type == "meta"]
    if on_meta or unexpected:
        raise RuntimeError(f"statetree_b200 load: uninitialised {on_meta[:5]}, unexpected {unexpected[:5]}")
    model.eval()
    return model
