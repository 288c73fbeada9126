"""Benchmark of the state-tree decode hot path on B200: the fused decode + GEMV / GEMM sweep over Qwen3-8B-shaped
linears (q/o 4096x4096, k/v 1024x4096, gate/up 12288x4096, down 4096x12288; 36 layers), synthetic seeded weights
N(0, 0.02) with 1% of the columns scaled x8.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--impl reference]

One step = every linear of all 36 layers once at batch M (default 1), captured in one CUDA graph.  All 36 layers own
distinct record buffers (10.5 GB in total, far beyond the 126 MB L2), so every step streams the records from HBM.
Launch layout of the step on one GPU: q / k / v and gate / up as fused trees, four launches per layer (the layout the
reference's conversion writes by default and its per-layer-kind GEMV table measures: qkv, o, gate_up, down); the
records of a layer's q, k, v (and gate, up) lie back to back, so the same buffers also serve as separate trees, and
the line reports the two other layouts beside it: one list launch per group over the separate trees
(`separate_trees_list_launches`, also `--lists`) and one launch per linear (`one_launch_per_linear`, `--per-linear`).
value    = algorithmic bytes (records + activations in + out) / device time, inputs resident in HBM
e2e      = the same through the C-ABI shim (statetree_b200.ops.ext().gemv / .gemm, the call TreeLinear.forward makes) with
           pinned host activations copied in and results copied out every step
roofline = the GEMV (or GEMM) kernel's achieved algorithmic GB/s against the measured HBM copy bandwidth
cpu_baseline / --impl reference = the reference's CPU path (decode + BF16 matmul) restated in C, on the host cores,
on a bounded sample (the linears of one layer).
With N > 1 ranks (torchrun) the linears are tensor-parallel: q/k/v and gate/up split by rows and stored per rank as
fused trees (four launches per layer), o/down split by columns, their GEMV adding the ranks' partial sums over NVLink
peer memory itself; total work is fixed (strong scaling).  Before timing, the all-reduced outputs of one layer
are checked against the fp64 product over the unsharded weights (`tp_check`).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "statetree-representation_b200"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)

LAYERS = 36
HIDDEN, INTER, KVDIM = 4096, 12288, 1024
# name, out rows, in cols, parallel kind ("col": rows split over ranks, "row": columns split + all-reduce)
SHAPES = [("q", HIDDEN, HIDDEN, "col"), ("k", KVDIM, HIDDEN, "col"), ("v", KVDIM, HIDDEN, "col"),
          ("o", HIDDEN, HIDDEN, "row"), ("gate", INTER, HIDDEN, "col"), ("up", INTER, HIDDEN, "col"),
          ("down", HIDDEN, INTER, "row")]
METRIC = "compressed GEMV/GEMM effective GB/s (Qwen3-8B linears, 36 layers)"


def algorithmic_bytes(M, N, B):
    """records + activations read + outputs written (the per-unit figure the roofline is computed from)"""
    return (M // 16) * (N // 64) * 1552 + 2 * B * N + 2 * B * M


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def measured_traffic(batch, world, layers, layout):
    """DRAM bytes per launch of the dominant kernel from the tracked ncu summary (a JSON next to the text summary that
    also names the kernel source it was captured from); (None, reason) when there is none for this workload or the
    kernel source has changed since the capture"""
    import hashlib
    path = os.path.join(ROOT, "profiles", "gemv_qwen3_8b_linears_b1.json")
    if not (batch == 1 and world == 1 and layers == LAYERS and os.path.exists(path)):
        return None, "no capture for this workload"
    with open(path) as f:
        rec = json.load(f)
    src = os.path.join(ROOT, "statetree-representation_b200", "csrc", "st_gemv.cu")
    with open(src, "rb") as f:
        sha = hashlib.sha256(f.read()).hexdigest()[:16]
    if rec.get("kernel_source_sha256_16") != sha:
        return None, "kernel source changed since the capture"
    if rec.get("layout") != layout:
        return None, "no capture for this launch layout"
    return rec["dram_bytes_per_launch"], f"ncu capture of {rec.get('captured', '?')}"


class ClockSampler:
    """samples nvidia-smi clocks and throttle reasons during the timed region"""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "25"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference(steps, warmup, batch):
    """the reference's CPU path (decode + BF16 matmul, restated in oracle/statetree_oracle.c) on the host cores;
    one step = the seven linears of ONE layer (1/36 of the GPU step)"""
    import numpy as np

    import gen_inputs as G
    import oracle
    oracle.build()
    oracle.set_threads(len(os.sched_getaffinity(0)))            # all the cores this process may use (torchrun sets 1)
    encs, xs = [], {}
    rs = np.random.RandomState(0)
    for name, M, N, _ in SHAPES:
        encs.append((name, M, N, oracle.encode(G.weights(M, N, len(encs), "llm"))))
        if N not in xs:
            xs[N] = G.to_bf16_bits(rs.standard_normal((batch, N)))
    scratch = np.empty(INTER * HIDDEN, dtype=np.uint16)
    nbytes = sum(algorithmic_bytes(M, N, batch) for _, M, N, _ in SHAPES)

    def step():
        for _, M, N, enc in encs:
            oracle.linear_cpu(enc, xs[N], scratch[:M * N].reshape(M, N))

    for _ in range(max(1, min(warmup, 1))):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return nbytes / dt / 1e9, dt, oracle.threads()


def attention_workload(args):
    """Decode attention over compressed KV pages (32 query / 8 KV heads, head_dim 128, 16-token pages; K = N(0,1) x
    per-channel LogNormal(0,1), V, q = N(0,1)), contexts 1K/4K/16K x batch 1/8/32/64, L2 flushed between calls, against
    BF16 attention over the same (exactly decoded) values.  Prints one JSON line with a table."""
    import math

    import torch

    from statetree_b200 import ops
    from statetree_b200.kvcache import PageStore, decode_splits

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    Hq, Hkv, D = 32, 8, 128
    try:
        from flash_attn import flash_attn_with_kvcache
        baseline_name = "flash_attn_with_kvcache (FlashAttention-2 %s, dense BF16 cache)" % __import__("flash_attn").__version__
    except Exception:                                         # noqa: BLE001
        flash_attn_with_kvcache = None
        baseline_name = "torch SDPA (enable_gqa) over a dense BF16 cache"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm, _, which = peaks()
    gen = torch.Generator(device=dev).manual_seed(0)
    table = []
    ctxs = [int(c) for c in args.ctx.split(",")]
    batches = [int(b) for b in args.attn_batch.split(",")]

    def timed(fn, reps):
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    for ctx in ctxs:
        for B in batches:
            npg = ctx // 16
            layer = PageStore(B * npg, Hkv, dev, pool_blocks=1 << 16)
            bt = torch.randperm(B * npg, device=dev, generator=gen).view(B, npg).to(torch.int32)
            scale_k = torch.exp(torch.randn(Hkv, D, device=dev, generator=gen))
            Kd = torch.empty(B, ctx, Hkv, D, dtype=torch.bfloat16, device=dev)
            Vd = torch.empty_like(Kd)
            pos = torch.arange(ctx, device=dev)
            for b in range(B):
                Kd[b] = (torch.randn(ctx, Hkv, D, device=dev, generator=gen) * scale_k).to(torch.bfloat16)
                Vd[b] = torch.randn(ctx, Hkv, D, device=dev, generator=gen).to(torch.bfloat16)
                slots = bt[b].long()[pos // 16] * 16 + pos % 16
                layer.append(Kd[b], Vd[b], slots)
            layer.check()
            q = torch.randn(B, Hq, D, device=dev, generator=gen).to(torch.bfloat16)
            lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
            S = decode_splits(B, Hkv, npg)
            sc = 1.0 / math.sqrt(D)
            out = torch.empty(B, Hq, D, dtype=torch.bfloat16, device=dev)
            ours = lambda: layer.attention(q, bt, lens, sc, splits=S, min_pages=4, out=out)   # noqa: E731
            if flash_attn_with_kvcache is not None:
                q4 = q.view(B, 1, Hq, D)
                base = lambda: flash_attn_with_kvcache(q4, Kd, Vd, cache_seqlens=lens, softmax_scale=sc)   # noqa: E731
            else:
                qs = q.view(B, Hq, 1, D)
                kt, vt = Kd.transpose(1, 2), Vd.transpose(1, 2)
                base = lambda: torch.nn.functional.scaled_dot_product_attention(qs, kt, vt, scale=sc, enable_gqa=True)   # noqa: E731
            for _ in range(3):
                ours()
                ref = base()
            err = float((out.float().view(-1) - ref.float().reshape(-1)).norm() / ref.float().norm())
            # correctness gate: the first two sequences against fp64 attention over the exactly decoded values
            worst = 0.0
            for b in range(min(B, 2)):
                k64 = Kd[b].double().permute(1, 0, 2).repeat_interleave(Hq // Hkv, 0)
                v64 = Vd[b].double().permute(1, 0, 2).repeat_interleave(Hq // Hkv, 0)
                p64 = torch.softmax(torch.einsum("hd,hld->hl", q[b].double(), k64) * sc, -1)
                r64 = torch.einsum("hl,hld->hd", p64, v64)
                worst = max(worst, float((out[b].double() - r64).norm() / r64.norm()))
                del k64, v64, p64, r64
            if not worst < 5e-3:
                raise RuntimeError(f"attention output off by {worst:.2e} (relative) from fp64 at batch {B}, context {ctx}")
            us, us_b = timed(ours, args.steps), timed(base, args.steps)
            nbytes = B * npg * 16 * Hkv * 400
            table.append({"batch": B, "ctx": ctx, "splits": S, "us": us, "bf16_us": us_b, "speedup_vs_bf16": us_b / us,
                          "gbs": nbytes / us / 1e3, "frac_hbm": nbytes / us / 1e3 / hbm, "rel_err_vs_bf16": err,
                          "rel_err_vs_fp64": worst})
            del layer, Kd, Vd
            torch.cuda.empty_cache()
    big = table[-1]
    print(json.dumps({"metric": "decode attention over compressed KV pages, effective GB/s (record bytes / time)",
                      "value": big["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": 3,
                      "ms_per_step": big["us"] / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "compressed-KV decode attention, 32q/8kv heads, d=128, 16-token pages; headline"
                                             f" row: batch {big['batch']} x ctx {big['ctx']}", "l2": "flushed between calls",
                                 "bf16_baseline": baseline_name},
                      "roofline": {"bound": "hbm", "achieved": big["gbs"], "peak": hbm, "unit": "GB/s",
                                   "frac": big["gbs"] / hbm, "traffic": None, "peak_source": f"of {which}"},
                      "device_status": ops.device_status(), "table": table}))


def moe_workload(args):
    """Routed-expert block of the Qwen3-30B-A3B shape (128 experts, top-8, hidden 2048, expert intermediate 768; all
    expert weights tree-stored): gate_up product -> SwiGLU gate -> down product -> routing-weighted sum for T tokens,
    uniform random routing, one CUDA graph per batch size, L2 flushed between replays.  Effective GB/s counts the
    records of the distinct (expert, projection) pairs actually read."""
    import torch

    import statetree_b200 as S
    from statetree_b200 import ops
    from statetree_b200.experts import TreeExperts

    import torch.distributed as dist

    from statetree_b200.parallel import expert_partition, peer_comm, reduce_partials

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        peer_comm()
    E, K, H, I = 128, 8, 2048, 768
    e_lo, e_hi, emap = expert_partition(E, rank, world, dev)   # expert parallel: this rank owns experts [e_lo, e_hi)
    gen = torch.Generator(device=dev).manual_seed(0)
    base13 = [S.TreeLinear.from_weight((torch.randn(2 * I, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16),
                                       verify=(i == 0)) for i in range(4)]
    base2 = [S.TreeLinear.from_weight((torch.randn(H, I, device=dev, generator=gen) * 0.02).to(torch.bfloat16),
                                      verify=(i == 0)) for i in range(4)]

    def clone(tl):
        c = S.TreeLinear(tl.in_features, tl.out_features, device="meta", n_esc=tl.esc_rows.numel())
        c._buffers["tree"] = tl.tree.clone()
        for k in ("esc_rows", "esc_cols", "esc_bits"):
            c._buffers[k] = tl._buffers[k]
        return c

    te = TreeExperts([clone(base13[e % 4]) for e in range(e_lo, e_hi)], [clone(base2[e % 4]) for e in range(e_lo, e_hi)])
    te.tables()
    if args.moe_no_gemm:
        import statetree_b200.experts as _X
        _X.GEMM_PAIRS_PER_EXPERT = 1 << 30
    else:
        te.tensor_maps()

    def block(x, ids, w):
        """every rank routes all tokens; pairs of other ranks' experts weigh zero; partial outputs are all-reduced"""
        if world == 1:
            return te(x, ids, w)
        out = te(x, ids, w, emap)
        reduce_partials(out)
        return out

    rec13, rec2 = base13[0].record_bytes(), base2[0].record_bytes()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm, _, which = peaks()
    table = []
    for T in [int(b) for b in args.moe_batch.split(",")]:
        x = torch.randn(T, H, device=dev, generator=gen).to(torch.bfloat16)
        w, ids = torch.softmax(torch.randn(T, E, device=dev, generator=gen), -1).topk(K, -1)
        w = (w / w.sum(-1, keepdim=True)).float().contiguous()
        ids = ids.to(torch.int32).contiguous()
        side = torch.cuda.Stream(dev)
        torch.cuda.synchronize()                                   # inputs were produced on the default stream
        with torch.cuda.stream(side):
            for _ in range(2):
                out = block(x, ids, w)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = block(x, ids, w)
        torch.cuda.synchronize()
        ts = []
        for _ in range(max(5, args.steps)):
            flush.zero_()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        us = ts[len(ts) // 2]
        if world > 1:
            t_ = torch.tensor([us], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            us = float(t_.item())
        # BF16 control: the same block with dense BF16 expert weights gathered per pair (batched matmul)
        distinct = int(ids.unique().numel())
        nbytes = distinct * (rec13 + rec2) + T * H * 2 * 2 + T * K * (2 * I + I + H) * 2
        ref = None
        if T * K <= 64 and world == 1:
            W13 = torch.stack([m.dequantize() for m in te.w13])
            W2 = torch.stack([m.dequantize() for m in te.w2])
            xe = x.repeat_interleave(K, 0).unsqueeze(2)

            def bf16_block():
                gu = torch.bmm(W13[ids.view(-1).long()], xe).squeeze(2)
                act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
                y = torch.bmm(W2[ids.view(-1).long()], act.unsqueeze(2)).squeeze(2)
                return (y.view(T, K, H).float() * w.unsqueeze(-1)).sum(1)

            ref = bf16_block()
            err = float((out.float() - ref).norm() / ref.norm())
            del W13, W2
        else:
            err = None
        table.append({"tokens": T, "pairs": T * K, "distinct_experts": distinct, "us": us, "gbs": nbytes / us / 1e3,
                      "frac_hbm": nbytes / us / 1e3 / hbm, "rel_err_vs_bf16": err})
        del graph
    big = table[0]
    status = ops.device_status()
    if rank != 0:
        sys.stdout.flush()
        os._exit(0)
    print(json.dumps({"metric": "MoE routed-expert block over tree-stored experts, effective GB/s (distinct expert records / time)",
                      "value": big["gbs"], "unit": "GB/s", "n_gpus": world, "steps": max(5, args.steps), "warmup": 2,
                      "ms_per_step": big["us"] / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"Qwen3-30B-A3B-shaped expert block: {E} experts top-{K}, hidden {H}, "
                                             f"intermediate {I}; headline row: {big['tokens']} token(s)",
                                 "l2": "flushed between replays",
                                 "parallelism": "single GPU" if world == 1 else f"ep{world} (experts split over ranks, "
                                                "tokens replicated, all-reduce of the partial outputs)"},
                      "roofline": {"bound": "hbm", "achieved": big["gbs"], "peak": hbm, "unit": "GB/s",
                                   "frac": big["gbs"] / hbm, "traffic": None, "peak_source": f"of {which}"},
                      "device_status": status, "table": table}))
    if world > 1:
        sys.stdout.flush()
        os._exit(0)


def aux_workload(args):
    """The streaming kernels beside the products: tree -> BF16 decode, embedding row gather, KV page append and
    dequant.  One JSON line with a table (median of L2-flushed calls)."""
    import torch

    import statetree_b200 as S
    from statetree_b200 import ops
    from statetree_b200.kvcache import PageStore

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm, _, which = peaks()
    gen = torch.Generator(device=dev).manual_seed(0)
    table = []

    def timed(fn):
        ts = []
        for _ in range(max(5, args.steps)):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    def row(name, us, nbytes):
        table.append({"kernel": name, "us": us, "gbs": nbytes / us / 1e3, "frac_hbm": nbytes / us / 1e3 / hbm})

    for M, N in ((4096, 4096), (12288, 4096)):
        W = (torch.randn(M, N, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        tl = S.TreeLinear.from_weight(W, verify=True)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        eo, el, _ = tl.tables()
        for _ in range(2):
            ops.ext().dec(tl.tree, eo, el, out)
        row(f"dec {M}x{N} (records read + BF16 written)", timed(lambda: ops.ext().dec(tl.tree, eo, el, out)),
            tl.record_bytes() + 2 * M * N)
        if M == 12288:
            ids = torch.randint(0, M, (64,), device=dev, generator=gen)
            for _ in range(2):
                tl.rows(ids)
            row("rows: 64 rows of a 12288x4096 table", timed(lambda: tl.rows(ids)), 64 * (N // 64) * 1552 + 64 * N * 2)
    H = 8
    for n_tok, what in ((64, "decode step, batch 64 (one token per sequence)"), (8192, "prefill, 8192 tokens")):
        layer = PageStore(max(64, n_tok // 16) * 2, H, dev, pool_blocks=1 << 14)
        K = torch.randn(n_tok, H, 128, device=dev, generator=gen).to(torch.bfloat16)
        V = torch.randn(n_tok, H, 128, device=dev, generator=gen).to(torch.bfloat16)
        slots = (torch.arange(n_tok, device=dev) * 16) if n_tok == 64 else torch.arange(n_tok, device=dev)
        for _ in range(2):
            layer.append(K, V, slots)
        row(f"kv_append: {what}", timed(lambda: layer.append(K, V, slots)), n_tok * H * (2 * 128 * 2 + 400))
        if n_tok == 8192:
            for _ in range(2):
                layer.dense()
            nb = layer.pages.shape[0]
            row(f"kv_dequant: {nb} pages", timed(lambda: layer.dense()), nb * H * (6400 + 8192))
        layer.check()
    big = table[1]
    print(json.dumps({"metric": "streaming kernels (dec, rows, kv_append, kv_dequant), effective GB/s", "value": big["gbs"],
                      "unit": "GB/s", "n_gpus": 1, "steps": max(5, args.steps), "warmup": 2, "ms_per_step": big["us"] / 1e3,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                      "config": {"workload": "dec / rows / kv_append / kv_dequant; headline row: " + big["kernel"],
                                 "l2": "flushed between calls"},
                      "roofline": {"bound": "hbm", "achieved": big["gbs"], "peak": hbm, "unit": "GB/s",
                                   "frac": big["gbs"] / hbm, "traffic": None, "peak_source": f"of {which}"},
                      "device_status": ops.device_status(), "table": table}))


def decode_workload(args):
    """Greedy decode with a random-init Qwen3-8B-architecture model (36 layers, hidden 4096, 32 q / 8 kv heads,
    head_dim 128, SwiGLU 12288, vocab 151936; weights N(0, 0.02)): uniform-random prompt tokens fed one step at a time,
    then greedy tokens, every step one CUDA-graph replay.  Compressed weights + compressed KV against the BF16 control
    built from the same seeds (dense weights, dense KV, FlashAttention).  Tensor-parallel when launched with N ranks."""
    import torch
    import torch.distributed as dist

    from statetree_b200 import ops
    from statetree_b200.decoder import DecoderConfig, TreeDecoder

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    moe = args.model == "qwen3-30b-a3b"
    if moe:                                                   # config 5: 48 layers, hidden 2048, 32 q / 4 kv heads, 128 experts top-8
        cfg = DecoderConfig(layers=48 if args.layers == LAYERS else args.layers, hidden=2048, heads=32, kv_heads=4,
                            inter=768, experts=128, top_k=8, moe_inter=768)
    else:
        cfg = DecoderConfig(layers=args.layers)
    B, P, Gn = args.batch, args.prompt, args.gen
    prompt = torch.randint(0, cfg.vocab, (B, P), generator=torch.Generator().manual_seed(1)).to(dev)
    res = {}
    for name, compressed in ((("statetree", True),) if moe else (("statetree", True), ("bf16", False))):
        m = TreeDecoder(cfg, dev, B, P + Gn + 16, compressed=compressed, seed=0, rank=rank, world=world)
        wbytes = m.weight_bytes()
        m.capture()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        preds = []
        margins = []
        toks = m.run(prompt, Gn, collect=preds, margins=margins)  # warm pass (also the token streams that are compared)
        m.reset()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        for t in range(P):
            m.tokens.copy_(prompt[:, t])
            m.graph.replay()
        e0.record()
        m.run(prompt[:, :0], Gn)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / Gn
        if world > 1:
            t_ = torch.tensor([ms], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            ms = float(t_.item())
        res[name] = {"ms_per_step": ms, "tok_s": B / (ms * 1e-3), "tokens": toks.cpu(), "weight_bytes_per_rank": wbytes,
                     "teacher_forced": torch.stack(preds, 1).cpu(),
                     "margins": torch.stack(margins).cpu() if margins else None}
        if compressed:
            m.cache.check()
        del m
        torch.cuda.empty_cache()
    st = res["statetree"]
    if moe:
        status = ops.device_status()
        if rank == 0:
            hbm, _, which = peaks()
            eff = st["weight_bytes_per_rank"] / (st["ms_per_step"] * 1e-3) / 1e9
            print(json.dumps({"metric": "greedy decode tokens/s, random-init Qwen3-30B-A3B architecture, compressed weights + KV",
                              "value": st["tok_s"], "unit": "tokens/s", "n_gpus": world, "steps": Gn, "warmup": P,
                              "ms_per_step": st["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                              "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                              "config": {"workload": f"Qwen3-30B-A3B-shape decode ({cfg.layers} layers, hidden 2048, 32 q / 4 kv "
                                                     f"heads, 128 experts top-8, expert intermediate 768), batch {B}, {P} random "
                                                     f"prompt tokens + {Gn} greedy tokens",
                                         "parallelism": "single GPU" if world == 1 else
                                         f"ep{world}: experts split over ranks, tokens replicated, partial outputs all-reduced; "
                                         f"attention tensor-parallel"},
                              "bf16_control": None,
                              "roofline": {"bound": "hbm", "achieved": eff, "peak": hbm, "unit": "GB/s", "frac": eff / hbm,
                                           "traffic": None, "peak_source": f"of {which}",
                                           "note": "record bytes a step reads per rank (upper bound for the experts) / step time"},
                              "device_status": status}))
        if world > 1:
            sys.stdout.flush()
            os._exit(0)
        return
    bf = res["bf16"]
    same = (st["tokens"] == bf["tokens"])
    first_div = [int((~same[b]).nonzero()[0]) if (~same[b]).any() else Gn for b in range(B)]
    # top-2 logit margin of the compressed model at the step where sequence 0's stream leaves the control's
    margin = None
    if first_div[0] < Gn and st["margins"] is not None:
        margin = float(st["margins"][first_div[0]])
    tf_same = float((st["teacher_forced"] == bf["teacher_forced"]).float().mean())
    status = ops.device_status()
    if rank == 0:
        hbm, _, which = peaks()
        eff = st["weight_bytes_per_rank"] / (st["ms_per_step"] * 1e-3) / 1e9
        print(json.dumps({"metric": "greedy decode tokens/s, random-init Qwen3-8B architecture, compressed weights + KV",
                          "value": st["tok_s"], "unit": "tokens/s", "n_gpus": world, "steps": Gn, "warmup": P,
                          "ms_per_step": st["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"Qwen3-8B-shape decode, {args.layers} layers, batch {B}, {P} prompt + {Gn} "
                                                 "greedy tokens", "parallelism": "single GPU" if world == 1 else f"tp{world}"},
                          "bf16_control": {"tok_s": bf["tok_s"], "ms_per_step": bf["ms_per_step"],
                                           "what": "same seeds: dense BF16 weights (cuBLAS), dense KV, FlashAttention-2"},
                          "speedup_vs_bf16": st["tok_s"] / bf["tok_s"],
                          "agreement_with_bf16": {"teacher_forced_top1": tf_same,
                                                  "greedy_fraction_equal": float(same.float().mean()),
                                                  "greedy_first_divergence_step_per_sequence": first_div,
                                                  "top2_logit_margin_at_first_divergence": margin,
                                                  "note": "random-init weights give nearly flat logits: a different fp32 "
                                                          "summation order flips near-ties, after which greedy streams differ"},
                          "roofline": {"bound": "hbm", "achieved": eff, "peak": hbm, "unit": "GB/s", "frac": eff / hbm,
                                       "traffic": None, "peak_source": f"of {which}",
                                       "note": "weight records per rank / step time (KV and activations not counted)"},
                          "device_status": status}))
    if world > 1:
        sys.stdout.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1, help="activation rows M (1, 8, 32, 64, 256)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-bf16", action="store_true", help="skip the dense BF16 (cuBLAS) control pass")
    ap.add_argument("--no-sweep", action="store_true", help="skip the M = 8 / 32 / 64 / 256 points of the default run")
    ap.add_argument("--no-fused", action="store_true", help="skip the extra passes over the other launch layouts")
    ap.add_argument("--separate-allreduce", action="store_true",
                    help="tensor parallel: o / down as a GEMV followed by the all-reduce kernel (two launches) instead of the "
                         "GEMV that sums over the ranks itself")
    ap.add_argument("--per-linear", action="store_true",
                    help="one GPU: one launch per linear (7 per layer) as the main step instead of q/k/v and gate/up as "
                         "fused trees (4 per layer)")
    ap.add_argument("--lists", action="store_true",
                    help="one GPU: q/k/v and gate/up as separate trees, one list launch per group, as the main step")
    ap.add_argument("--moe-batch", default="1,8,32,64,512,2048")
    ap.add_argument("--moe-no-gemm", action="store_true", help="moe workload: grouped GEMV at every size (for comparison)")
    ap.add_argument("--model", default="qwen3-8b", choices=["qwen3-8b", "qwen3-30b-a3b"],
                    help="decode workload: the dense Qwen3-8B shape (config 4) or the Qwen3-30B-A3B mixture of experts (config 5)")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--gen", type=int, default=512)
    ap.add_argument("--workload", default="linear", choices=["linear", "attn", "moe", "decode", "aux"],
                    help="linear: the Qwen3-8B linear sweep (default, the headline); attn: compressed-KV decode attention")
    ap.add_argument("--ctx", default="1024,4096,16384")
    ap.add_argument("--attn-batch", default="1,8,32,64")
    args = ap.parse_args()
    if args.workload == "decode":
        decode_workload(args)
        return
    if args.workload == "moe":
        moe_workload(args)
        return
    if args.workload == "aux":
        if int(os.environ.get("RANK", "0")) == 0:
            aux_workload(args)
        return
    if args.workload == "attn":
        if int(os.environ.get("RANK", "0")) == 0:
            attention_workload(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": f"Qwen3-8B-shaped linears (q/o 4096x4096, k/v 1024x4096, gate/up 12288x4096, down 4096x12288)"
                          f" x {args.layers} layers, batch M={args.batch}, seeds per shape, N(0,0.02) + 1% columns x8",
              "batch": args.batch, "layers": args.layers,
              "l2": "inputs larger than L2: 10.5 GB of distinct record buffers per step",
              "parallelism": ("single GPU, one launch per linear (7 per layer)" if args.per_linear else
                              "single GPU; the seven trees of a layer in four launches: q/k/v and gate/up (separate trees, "
                              "shared input) as one list launch each, o and down one launch each" if args.lists else
                              "single GPU; q/k/v and gate/up stored as fused trees, the layout the reference's conversion "
                              "writes (DEFAULT_FUSE) and its per-layer-kind GEMV table measures: 4 launches per layer "
                              "(qkv 6144x4096, o, gate_up 24576x4096, down)") if world == 1 else
              f"tp{world} (q/k/v and gate/up of a rank as fused trees; o/down column shards whose GEMV adds the ranks' "
              "fp32 tile sums over NVLink peer memory itself: four launches per layer and rank)"}

    if args.impl == "reference":
        if rank != 0:
            return
        steps = max(1, min(args.steps, 5))
        val, dt, cores = cpu_reference(steps, args.warmup, args.batch)
        sample = "the seven linears of one layer per step (1/36 of the GPU step's work)"
        print(json.dumps({"metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
                          "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "impl": "reference", "config": config,
                          "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
                          "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch
    import torch.distributed as dist

    import statetree_b200 as S
    from statetree_b200 import ops
    from statetree_b200.linear import GEMV_MAX, _state
    from statetree_b200.parallel import peer_comm, reduce_partials

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = peer_comm()                             # IPC set-up of the peer-memory exchange, outside any capture
    E = ops.ext()
    B = args.batch
    assert 1 <= B <= 4096

    # ---- weights: the seven matrices from their seeds; one encoded set per launch (this rank's shard), cloned into
    # `layers` distinct record buffers.  One GPU: the seven linears as seven launches.  Tensor parallel: q/k/v and
    # gate/up of a rank stored as fused trees (four launches per layer), o and down split by columns.
    gen = torch.Generator(device=dev)
    full = {}
    for i, (name, M, N, kind) in enumerate(SHAPES):
        gen.manual_seed(i)
        W = torch.randn(M, N, device=dev, generator=gen) * 0.02
        cols = torch.randperm(N, device=dev, generator=gen)[:N // 100]
        W[:, cols] *= 8.0
        full[name] = W.to(torch.bfloat16)
        del W

    def rows_of(name):
        W = full[name]
        per = W.shape[0] // world
        return W[rank * per:(rank + 1) * per]

    def cols_of(name):
        W = full[name]
        per = W.shape[1] // world
        return W[:, rank * per:(rank + 1) * per].contiguous()

    Hs, Is = HIDDEN // world, INTER // world                 # o's / down's input columns on this rank
    x_h = torch.randn(B, HIDDEN, generator=torch.Generator().manual_seed(100)).to(torch.bfloat16).pin_memory()
    x2_h = torch.randn(B, INTER, generator=torch.Generator().manual_seed(101)).to(torch.bfloat16).pin_memory()
    x = x_h.to(dev)
    x_o = x_h[:, rank * Hs:(rank + 1) * Hs].contiguous().to(dev)
    x_d = x2_h[:, rank * Is:(rank + 1) * Is].contiguous().to(dev)
    if world == 1:
        plan = [(n, full[n], {"o": x_o, "down": x_d}.get(n, x), k) for n, _, _, k in SHAPES]
    else:
        plan = [("qkv", torch.cat([rows_of("q"), rows_of("k"), rows_of("v")]), x, "col"), ("o", cols_of("o"), x_o, "row"),
                ("gate_up", torch.cat([rows_of("gate"), rows_of("up")]), x, "col"), ("down", cols_of("down"), x_d, "row")]
    shard = [S.TreeLinear.from_weight(W.contiguous(), verify=(i == 0)) for i, (_, W, _, _) in enumerate(plan)]
    ins = [xin for _, _, xin, _ in plan]
    kinds = [k for _, _, _, k in plan]
    layers, fbufs = [], []
    groups = [(0, 3), (4, 6)] if world == 1 else []          # q / k / v and gate / up: stored back to back per layer
    for _ in range(args.layers):
        trees = [None] * len(shard)
        bufs = []
        for lo, hi in groups:                                # one buffer per group; the members' trees are views into it
            buf = torch.cat([shard[i].tree for i in range(lo, hi)])
            at = 0
            for i in range(lo, hi):
                n = shard[i].tree.shape[0]
                trees[i] = buf[at:at + n]
                at += n
            bufs.append(buf)
        row = []
        for i, tl in enumerate(shard):
            c = S.TreeLinear(tl.in_features, tl.out_features, device="meta", n_esc=tl.esc_rows.numel())
            c._buffers["tree"] = trees[i] if trees[i] is not None else tl.tree.clone()
            for k in ("esc_rows", "esc_cols", "esc_bits"):
                c._buffers[k] = tl._buffers[k]
            c._tables = tl.tables()
            row.append(c)
        layers.append(row)
        fbufs.append(bufs)
    torch.cuda.synchronize()

    outs = [torch.empty(B, tl.out_features, dtype=torch.bfloat16, device=dev) for tl in layers[0]]
    outs_h = [torch.empty(o.shape, dtype=torch.bfloat16).pin_memory() for o in outs]
    launches = 0
    use_gemv = B <= GEMV_MAX
    st = _state(dev)
    ws_need = max((E.gemv_workspace_bytes if use_gemv else E.gemm_workspace_bytes)(tl.out_features, tl.in_features, B)
                  for tl in layers[0])
    use_lists = world == 1                                   # (the list and fused variants exist on one GPU)
    main_mode = "per_linear" if (world > 1 or args.per_linear) else ("lists" if args.lists else "fused")
    Mq, Mg = (sum(tl.out_features for tl in layers[0][0:3]), sum(tl.out_features for tl in layers[0][4:6])) if world == 1 else (0, 0)
    if world == 1:
        wsb = E.gemv_workspace_bytes if use_gemv else E.gemm_workspace_bytes
        ws_need = max(ws_need, wsb(Mq, HIDDEN, B), wsb(Mg, HIDDEN, B))
        if use_gemv:
            ws_need = max(ws_need, E.gemv_list_workspace_bytes([tl.out_features for tl in layers[0][0:3]], HIDDEN, B),
                          E.gemv_list_workspace_bytes([tl.out_features for tl in layers[0][4:6]], HIDDEN, B))
    ws = st.get_ws(ws_need) if use_gemv else st.get_scratch(ws_need)   # (the GEMM's workspace is plain scratch)
    cnt = st.get_cnt(4096)
    # escape tables of the fused trees (the members' lists with their rows shifted)
    ftabs, fouts, fouts_h = None, None, None
    if world == 1:
        from statetree_b200 import format as F

        def fuse(tls):
            rows, off = [], 0
            for t in tls:
                rows.append(t.esc_rows + off)
                off += t.out_features
            return F.escape_tables(off, tls[0].in_features, torch.cat(rows), torch.cat([t.esc_cols for t in tls]),
                                   torch.cat([t.esc_bits for t in tls]))

        ftabs = (fuse(layers[0][0:3]), fuse(layers[0][4:6]))
        fouts = [torch.empty(B, Mq, dtype=torch.bfloat16, device=dev), torch.empty(B, Mg, dtype=torch.bfloat16, device=dev)]
        fouts_h = [torch.empty(o.shape, dtype=torch.bfloat16).pin_memory() for o in fouts]
        torch.cuda.synchronize()

    def list_args(row, lo, hi):
        tabs = []
        for tl in row[lo:hi]:
            eo, el, eb = tl._tables
            tabs.append((tl.tree, eo, eb, el))
        return E.gemv_list_args(tabs, outs[lo:hi])

    lists = [(list_args(row, 0, 3), list_args(row, 4, 6)) for row in layers] if use_lists else None

    def one(tl, xin, y):
        eo, el, eb = tl._tables
        if use_gemv:
            E.gemv(tl.tree, eo, eb, el, xin, y, ws, cnt)
        else:
            E.gemm(tl.tree, eo, el, xin, y, ws, cnt)

    fused_ar = (world > 1 and use_gemv and comm is not None and not args.separate_allreduce
                and comm.gemv_allreduce_fits(HIDDEN, B))

    def row_parallel(tl, xin, y):
        """o / down on this rank's column shard, summed over the ranks: returns the launches it took"""
        if fused_ar:
            eo, el, eb = tl._tables
            comm.gemv_allreduce(tl.tree, eo, eb, el, xin, y, ws)
            return 1
        one(tl, xin, y)
        reduce_partials(y)
        return 2                                             # the peer-memory all-reduce is one kernel of this library

    # ---- tensor-parallel check (before any timing): the all-reduced outputs of the row-parallel projections of one
    # layer against the fp64 product over the unsharded weights, and the same bits on every rank
    tp_check = None
    if world > 1:
        worst = 0.0
        for (name, _, xin, kind), tl, y in zip(plan, shard, outs):
            if kind != "row":
                continue
            row_parallel(tl, xin, y)
            xf = (x_h if name == "o" else x2_h).to(dev).double()
            ref = xf @ full[name].double().t()
            err = float((y.double() - ref).norm() / ref.norm())
            worst = max(worst, err)
            gathered = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(gathered, y)
            same = all(torch.equal(g.view(torch.int16), y.view(torch.int16)) for g in gathered)
            if not (err < 5e-3 and same):
                raise RuntimeError(f"tensor-parallel check failed for {name}: rel. error {err:.2e} vs fp64, identical on "
                                   f"all ranks: {same}")
        tp_check = {"result": "ok", "max_rel_err_vs_fp64": worst, "bar": 5e-3,
                    "what": "all-reduced o and down outputs of one layer (BF16) against the fp64 product over the "
                            "unsharded weights; bit-identical on every rank",
                    "kernel": "gemv_kernel that adds the ranks' sums itself" if fused_ar else "gemv_kernel + allreduce_kernel"}
    del shard

    def run_lists():
        # q / k / v and gate / up read the same activations: each group is one launch over the members' trees
        for row, (qkv, gate_up) in zip(layers, lists):
            if use_gemv:
                E.gemv_list(qkv, x, ws)
            else:
                E.gemm_list(qkv, x, cnt)
            one(row[3], ins[3], outs[3])
            if use_gemv:
                E.gemv_list(gate_up, x, ws)
            else:
                E.gemm_list(gate_up, x, cnt)
            one(row[6], ins[6], outs[6])
        return 4 * len(layers)

    def fused_one(tree, tabs, y):
        eo, el, eb = tabs
        if use_gemv:
            E.gemv(tree, eo, eb, el, x, y, ws, cnt)
        else:
            E.gemm(tree, eo, el, x, y, ws, cnt)

    def run_fused():
        # q / k / v and gate / up of a layer are one tree each (their records lie back to back): four launches per layer
        for row, (qkv_buf, gu_buf) in zip(layers, fbufs):
            fused_one(qkv_buf, ftabs[0], fouts[0])
            one(row[3], ins[3], outs[3])
            fused_one(gu_buf, ftabs[1], fouts[1])
            one(row[6], ins[6], outs[6])
        return 4 * len(layers)

    def run_per_linear():
        n = 0
        for row in layers:
            for tl, xin, y, kind in zip(row, ins, outs, kinds):
                if world > 1 and kind == "row":
                    n += row_parallel(tl, xin, y)
                else:
                    one(tl, xin, y)
                    n += 1
        return n

    variants = {"fused": run_fused, "lists": run_lists, "per_linear": run_per_linear}
    run_layers = variants[main_mode]
    main_outs = ([fouts[0], outs[3], fouts[1], outs[6]], [fouts_h[0], outs_h[3], fouts_h[1], outs_h[6]]) if main_mode == "fused" else (outs, outs_h)

    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        launches = run_layers()                             # warm: function attributes, NCCL channels
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        run_layers()
    torch.cuda.synchronize()
    step_bytes = sum(algorithmic_bytes(M, N, B) for _, M, N, _ in SHAPES) * args.layers   # whole job, all ranks
    step_flops = sum(2 * B * M * N for _, M, N, _ in SHAPES) * args.layers

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def dev_step():
        graph.replay()

    def e2e_step():
        x.copy_(x_h, non_blocking=True)
        x_o.copy_(x_h[:, rank * Hs:(rank + 1) * Hs], non_blocking=True)
        x_d.copy_(x2_h[:, rank * Is:(rank + 1) * Is], non_blocking=True)
        graph.replay()
        for o, oh in zip(*main_outs):
            oh.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()            # the caller reads the result every step

    for _ in range(max(3, args.warmup)):
        dev_step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(dev_step, args.steps)
    for _ in range(2):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    # ---- the same bytes through the other launch layouts (one GPU): fused trees, list launches, one launch per linear
    WHAT = {"fused": ("fused_qkv_gate_up", "q/k/v and gate/up as fused trees (6144x4096, 24576x4096), the layout the "
                      "reference's conversion writes: 4 launches per layer", 4),
            "lists": ("separate_trees_list_launches", "q/k/v and gate/up as separate trees, one list launch per group: "
                      "4 launches per layer", 4),
            "per_linear": ("one_launch_per_linear", "separate trees, one launch per linear: 7 per layer", 7)}
    others = {}
    if world == 1 and not args.no_fused:
        for mode, fn in variants.items():
            if mode == main_mode:
                continue
            with torch.cuda.stream(side):
                fn()
            side.synchronize()
            vg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(vg, stream=side):
                fn()
            torch.cuda.synchronize()
            for _ in range(3):
                vg.replay()
            ms_v = timed(vg.replay, args.steps)
            key, what, per_layer = WHAT[mode]
            others[key] = {"what": what, "ms_per_step": ms_v, "value": step_bytes / (ms_v * 1e-3) / 1e9, "unit": "GB/s",
                           "frac": step_bytes / (ms_v * 1e-3) / 1e9 / peaks()[0],
                           "gpu_launches": per_layer * args.layers * args.steps}
            del vg
    # ---- BF16 control: the same step over dense BF16 copies of the same weights through torch.matmul (cuBLAS), the
    # comparison the reference's per-layer GEMV table makes (RESULTS.md:176-183); 36 distinct buffers per shape as above
    control = None
    if world == 1 and not args.no_bf16:
        # dense copies in the fused layout; the separate q / k / v and gate / up weights are row slices of them
        dense_f, dense = [], []
        for row, (qkv_buf, gu_buf) in zip(layers, fbufs):
            Wqkv = torch.empty(Mq, HIDDEN, dtype=torch.bfloat16, device=dev)
            Wgu = torch.empty(Mg, HIDDEN, dtype=torch.bfloat16, device=dev)
            E.dec(qkv_buf, ftabs[0][0], ftabs[0][1], Wqkv)
            E.dec(gu_buf, ftabs[1][0], ftabs[1][1], Wgu)
            Wo, Wd = row[3].dequantize(), row[6].dequantize()
            dense_f.append([Wqkv, Wo, Wgu, Wd])
            sep, at = [], 0
            for tl in row[0:3]:
                sep.append(Wqkv[at:at + tl.out_features])
                at += tl.out_features
            sep.append(Wo)
            at = 0
            for tl in row[4:6]:
                sep.append(Wgu[at:at + tl.out_features])
                at += tl.out_features
            sep.append(Wd)
            dense.append(sep)
        fused_main = main_mode == "fused"

        def control_fn(xs_, ys_, fys_):
            """the control in the launch layout of the main step: 4 matmuls per layer over fused weights, or 7"""
            if fused_main:
                def run():
                    for Wqkv, Wo, Wgu, Wd in dense_f:
                        torch.matmul(xs_[0], Wqkv.t(), out=fys_[0])
                        torch.matmul(xs_[1], Wo.t(), out=ys_[3])
                        torch.matmul(xs_[0], Wgu.t(), out=fys_[1])
                        torch.matmul(xs_[2], Wd.t(), out=ys_[6])
                return run

            def run():
                for row_d in dense:
                    for W, xin, y in zip(row_d, [xs_[0]] * 3 + [xs_[1]] + [xs_[0]] * 2 + [xs_[2]], ys_):
                        torch.matmul(xin, W.t(), out=y)
            return run

        def graph_time(fn, steps):
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn()
            torch.cuda.synchronize()
            for _ in range(3):
                g.replay()
            t = timed(g.replay, steps)
            del g
            return t

        douts = [torch.empty_like(o) for o in outs]
        dfouts = [torch.empty_like(o) for o in fouts]
        ms_d = graph_time(control_fn([x, x_o, x_d], douts, dfouts), args.steps)
        control = {"what": "same step in the same launch layout (" + ("4 matmuls per layer over fused weights"
                                                                       if fused_main else "7 matmuls per layer")
                           + "), dense BF16 copies of the same weights, torch.matmul (cuBLAS) in one CUDA graph",
                   "ms_per_step": ms_d, "speedup_vs_bf16": ms_d / ms}
        if fused_main:                                       # the control with one matmul per linear, for the other layouts
            fused_main = False
            ms_d7 = graph_time(control_fn([x, x_o, x_d], douts, dfouts), args.steps)
            fused_main = True
            control["ms_per_step_one_matmul_per_linear"] = ms_d7
        # ---- the other activation-row counts of the benchmark configuration (M = 8, 32, 64, 256), each one graph over the
        # same record buffers in the launch layout of the main step and one over the dense copies: a few replays each
        sweep = []
        if B == 1 and not args.no_sweep:
            for Bs in (8, 32, 64, 256):
                gs = torch.Generator(device=dev).manual_seed(200 + Bs)
                xs = [torch.randn(Bs, n, device=dev, generator=gs).to(torch.bfloat16) for n in (HIDDEN, HIDDEN, INTER)]
                ys = [torch.empty(Bs, tl.out_features, dtype=torch.bfloat16, device=dev) for tl in layers[0]]
                fys = [torch.empty(Bs, Mq, dtype=torch.bfloat16, device=dev), torch.empty(Bs, Mg, dtype=torch.bfloat16, device=dev)]
                gemv_path = Bs <= GEMV_MAX
                wsb = E.gemv_workspace_bytes if gemv_path else E.gemm_workspace_bytes
                need_s = max([wsb(tl.out_features, tl.in_features, Bs) for tl in layers[0]] + [wsb(Mq, HIDDEN, Bs), wsb(Mg, HIDDEN, Bs)])
                if gemv_path:
                    need_s = max(need_s, E.gemv_list_workspace_bytes([tl.out_features for tl in layers[0][0:3]], HIDDEN, Bs),
                                 E.gemv_list_workspace_bytes([tl.out_features for tl in layers[0][4:6]], HIDDEN, Bs))
                ws_s = st.get_ws(need_s) if gemv_path else st.get_scratch(need_s)
                cnt_s = st.get_cnt(4096)

                def mm(tree, tabs, xin, y):
                    eo, el, eb = tabs
                    if gemv_path:
                        E.gemv(tree, eo, eb, el, xin, y, ws_s, cnt_s)
                    else:
                        E.gemm(tree, eo, el, xin, y, ws_s, cnt_s)

                def largs(row, lo, hi):
                    tabs = []
                    for tl in row[lo:hi]:
                        eo, el, eb = tl._tables
                        tabs.append((tl.tree, eo, eb, el))
                    return E.gemv_list_args(tabs, ys[lo:hi])

                lists_s = [(largs(row, 0, 3), largs(row, 4, 6)) for row in layers] if main_mode == "lists" else None

                def run_tree():
                    for li, row in enumerate(layers):
                        if main_mode == "fused":
                            mm(fbufs[li][0], ftabs[0], xs[0], fys[0])
                            mm(row[3].tree, row[3]._tables, xs[1], ys[3])
                            mm(fbufs[li][1], ftabs[1], xs[0], fys[1])
                            mm(row[6].tree, row[6]._tables, xs[2], ys[6])
                        elif main_mode == "lists":
                            for k, grp in enumerate(lists_s[li]):
                                if gemv_path:
                                    E.gemv_list(grp, xs[0], ws_s)
                                else:
                                    E.gemm_list(grp, xs[0], cnt_s)
                                mm(row[3 + 3 * k].tree, row[3 + 3 * k]._tables, xs[1 + k], ys[3 + 3 * k])
                        else:
                            for tl, xin, y in zip(row, [xs[0]] * 3 + [xs[1]] + [xs[0]] * 2 + [xs[2]], ys):
                                mm(tl.tree, tl._tables, xin, y)

                kern = "gemv_kernel" if gemv_path else "gemm_kernel (tcgen05)"
                point = {"batch": Bs, "kernel": kern, "layout": main_mode}
                point["ms_per_step"] = graph_time(run_tree, 5)
                point["bf16_control_ms"] = graph_time(control_fn(xs, ys, fys), 5)
                nb = sum(algorithmic_bytes(M, N, Bs) for _, M, N, _ in SHAPES) * args.layers
                fl = sum(2 * Bs * M * N for _, M, N, _ in SHAPES) * args.layers
                point.update(gbs=nb / (point["ms_per_step"] * 1e-3) / 1e9, tflops=fl / (point["ms_per_step"] * 1e-3) / 1e12,
                             speedup_vs_bf16=point["bf16_control_ms"] / point["ms_per_step"])
                sweep.append(point)
                del xs, ys, fys
            control["sweep"] = sweep
        # ---- prefill-size batches (512 / 1024 / 2048 / 4096 rows): the two ways the tree-stored layers can run them, the
        # tcgen05 kernel (every token tile decodes the records again) and decode once + cuBLAS with the next layer
        # decoded on a side stream meanwhile (what TreeLinear does above PREFILL_MIN rows), against cuBLAS over the
        # dense copies.  Eager launches: a launch takes tens of microseconds of device time here
        prefill = []
        if B == 1 and not args.no_sweep and main_mode == "fused":
            import weakref

            def shell(tree, tabs, M, N):
                c = S.TreeLinear(N, M, device="meta")
                c._buffers["tree"] = tree
                c._tables = tabs
                return c

            chain = []
            for row, (qkv_buf, gu_buf) in zip(layers, fbufs):
                chain += [shell(qkv_buf, ftabs[0], Mq, HIDDEN), row[3], shell(gu_buf, ftabs[1], Mg, HIDDEN), row[6]]
            for a_, b_ in zip(chain, chain[1:] + chain[:1]):
                a_.__dict__["_next"] = weakref.ref(b_)
            for Bs in (512, 1024, 2048, 4096):
                gs = torch.Generator(device=dev).manual_seed(300 + Bs)
                xs = [torch.randn(Bs, n, device=dev, generator=gs).to(torch.bfloat16) for n in (HIDDEN, HIDDEN, INTER)]
                ys = [torch.empty(Bs, m, dtype=torch.bfloat16, device=dev) for m in (Mq, HIDDEN, Mg, HIDDEN)]
                xin4 = [xs[0], xs[1], xs[0], xs[2]]
                ws_p = st.get_scratch(max(E.gemm_workspace_bytes(m, n, Bs) for m, n in
                                          ((Mq, HIDDEN), (HIDDEN, HIDDEN), (Mg, HIDDEN), (HIDDEN, INTER))))
                cnt_p = st.get_cnt(4096)

                def run_kernel():
                    for i, tl in enumerate(chain):
                        eo, el, eb = tl._tables
                        E.gemm(tl.tree, eo, el, xin4[i % 4], ys[i % 4], ws_p, cnt_p)

                def run_dense_stage():
                    for i, tl in enumerate(chain):
                        st.dense_stage().run(tl, xin4[i % 4], ys[i % 4])

                def run_control():
                    for Wqkv, Wo, Wgu, Wd in dense_f:
                        torch.matmul(xs[0], Wqkv.t(), out=ys[0])
                        torch.matmul(xs[1], Wo.t(), out=ys[1])
                        torch.matmul(xs[0], Wgu.t(), out=ys[2])
                        torch.matmul(xs[2], Wd.t(), out=ys[3])

                def eager_time(fn):
                    fn()
                    torch.cuda.synchronize()
                    return timed(fn, 3)

                fl = sum(2 * Bs * M * N for _, M, N, _ in SHAPES) * args.layers
                t_k, t_d, t_c = eager_time(run_kernel), eager_time(run_dense_stage), eager_time(run_control)
                prefill.append({"batch": Bs, "tcgen05_kernel_ms": t_k, "decode_plus_cublas_ms": t_d, "bf16_control_ms": t_c,
                                "tflops_decode_plus_cublas": fl / (t_d * 1e-3) / 1e12,
                                "speedup_vs_bf16": t_c / min(t_k, t_d)})
                del xs, ys
            control["prefill"] = prefill
        del dense, dense_f
    status = ops.device_status()

    def leave():
        """multi-rank exit: the captured graph holds NCCL work, and tearing the process group down under it can block;
        every rank is past its last collective here, so flush and leave the process directly"""
        if world > 1:
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    if rank != 0:
        leave()
        return

    hbm, tf, which = peaks()
    value = step_bytes / (ms * 1e-3) / 1e9
    per_gpu = value / world
    traffic, traffic_source = measured_traffic(B, world, args.layers, main_mode)
    roof = {"bound": "hbm", "achieved": per_gpu, "peak": hbm, "unit": "GB/s", "frac": per_gpu / hbm,
            "traffic": traffic, "traffic_source": traffic_source, "peak_source": f"of {which}",
            "frac_of_nominal_8TBs": per_gpu / 8000.0,
            "kernel": "gemv_kernel" if use_gemv else "gemm_kernel",
            "bytes_per_launch": step_bytes / world / launches, "us_per_launch": ms * 1e3 / launches}
    if not use_gemv:
        roof["tensor_tflops"] = step_flops / world / (ms * 1e-3) / 1e12
        roof["tensor_frac"] = roof["tensor_tflops"] / tf
    line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config, "clocks": clocks,
            "e2e": {"value": step_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": 2 * B * (HIDDEN + Hs + Is),
                    "d2h_bytes_per_step": sum(o.numel() * 2 for o in outs)},
            "gpu_launches": launches * args.steps, "roofline": roof, "device_status": status,
            "bf16_equivalent_gbs": value * 16.0 / 12.125}
    if tp_check is not None:
        line["tp_check"] = tp_check
    line.update(others)
    if control is not None:
        if "sweep" in control:
            line["sweep"] = control.pop("sweep")
        if control.get("prefill"):
            line["prefill"] = control.pop("prefill")
        line["bf16_control"] = control
    if not args.no_cpu and world == 1:
        val, dt, cores = cpu_reference(2, 1, B)
        line["cpu_baseline"] = {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                                "sample": "the seven linears of one layer, 2 timed passes (1/36 of a GPU step each)"}
    print(json.dumps(line))
    leave()


if __name__ == "__main__":
    main()
