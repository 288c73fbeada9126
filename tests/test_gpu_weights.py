"""GPU parity of the weight kernels (dec, rows, GEMV, tcgen05 GEMM) against the CPU oracle, through the C ABI.

Bars: decoded weights bit-exact; fp32 accumulators within 1e-3 relative Frobenius error of the fp64 product over the
exactly decoded BF16 values (the BF16 output then carries only its own rounding: it must equal the rounded
accumulator); one-hot activations read columns of W back bit for bit; reruns are bit-identical.
"""
import os

import numpy as np
import pytest
import torch

import gen_inputs as G
import oracle
from util import bits_to_torch, layer_from_oracle, rel_fro, torch_to_bits

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 1e-3            # relative Frobenius error of fp32 accumulators against the fp64 product


def _status_ok():
    from statetree_b200 import ops
    assert ops.device_status() == 0


@pytest.mark.parametrize("name", ["mixed", "heavy", "each", "llm"])
def test_dec_of_reference_trees_is_exact(name):
    from statetree_b200 import TreeLinear
    g = np.load(os.path.join(GOLD, "weights_small.npz"))
    W = g[f"{name}_W"]
    M, N = W.shape
    tl = TreeLinear(N, M, device="meta", n_esc=g[f"{name}_esc_rows"].size)
    for k in ("tree", "esc_rows", "esc_cols", "esc_bits"):
        tl._buffers[k] = torch.from_numpy(g[f"{name}_{k}"]).to(DEV)
    assert np.array_equal(torch_to_bits(tl.dequantize()), W)


@pytest.mark.parametrize("M,N,seed,regime", [(256, 512, 0, "mixed"), (512, 1024, 1, "mixed"), (256, 2048, 5, "heavy"),
                                             (1024, 512, 6, "each"), (512, 768, 7, "llm"), (16, 64, 8, "mixed")])
def test_encode_on_gpu_equals_oracle_and_dec_roundtrips(M, N, seed, regime):
    from statetree_b200 import TreeLinear, format as F
    W = G.weights(M, N, seed, regime)
    enc = oracle.encode(W)
    Wt = bits_to_torch(W, DEV)
    got = F.encode(Wt)
    assert np.array_equal(got["tree"].cpu().numpy(), enc["tree"])
    for k in ("esc_rows", "esc_cols", "esc_bits"):
        assert np.array_equal(got[k].cpu().numpy(), enc[k])
    tl = TreeLinear.from_weight(Wt, verify=True)             # verify runs the dec kernel
    assert np.array_equal(torch_to_bits(tl.dequantize()), W)
    ids = torch.tensor([[0, M - 1, 17 % M], [5 % M, 5 % M, M // 2]], device=DEV)
    rows = tl.rows(ids)
    assert rows.shape == (2, 3, N)
    assert np.array_equal(torch_to_bits(rows).reshape(-1, N), W[ids.cpu().numpy().reshape(-1)])


def _check_linear(tl, W, B, seed, path):
    from statetree_b200.linear import _state
    rs = np.random.RandomState(seed)
    X = G.to_bf16_bits(rs.standard_normal((B, W.shape[1])))
    x = bits_to_torch(X, DEV)
    yf = torch.empty(B, W.shape[0], dtype=torch.float32, device=DEV)
    y = tl._forward(x, yf)
    torch.cuda.synchronize()
    ref = oracle.linear_f64(W, X)
    e32 = rel_fro(yf.cpu().numpy(), ref)
    assert e32 < TOL, (path, W.shape, B, e32)
    assert torch.equal(y, yf.to(torch.bfloat16)), (path, "BF16 output is not the rounded accumulator")
    e16 = rel_fro(y.float().cpu().numpy(), ref)
    assert e16 < 5e-3, (path, W.shape, B, e16)
    for _ in range(2):                                                     # bit-identical from run to run
        assert torch.equal(tl(x), y), (path, W.shape, B, "nondeterministic")
    st = _state(torch.device(DEV))
    assert int(st.cnt.abs().sum()) == 0                                   # semaphores left at zero
    return e32


@pytest.mark.parametrize("M,N,regime", [(512, 1024, "mixed"), (1024, 512, "mixed"), (256, 2048, "heavy"),
                                        (128, 768, "each"), (16, 64, "mixed"), (2048, 4096, "llm")])
def test_gemv_matches_fp64(M, N, regime, monkeypatch):
    import statetree_b200.linear as L
    monkeypatch.setattr(L, "GEMV_MAX", 32)                      # every batch here through the GEMV kernel (NT = 1, 2, 4)
    W = G.weights(M, N, M + N, regime)
    tl, _ = layer_from_oracle(W)
    for B in (1, 3, 8, 12, 16, 24, 32):
        _check_linear(tl, W, B, B, "gemv")
    _status_ok()


@pytest.mark.parametrize("M,N,regime", [(512, 1024, "mixed"), (1024, 512, "mixed"), (256, 2048, "heavy"),
                                        (128, 768, "each"), (2048, 4096, "llm"), (1280, 64, "mixed"),
                                        (1280, 192, "mixed"), (5120, 256, "mixed"), (128, 64, "mixed")])
def test_gemm_matches_fp64(M, N, regime, monkeypatch):
    import statetree_b200.linear as L
    monkeypatch.setattr(L, "PREFILL_MIN", 0)                    # every batch here through the tcgen05 kernel
    W = G.weights(M, N, M + N + 1, regime)
    tl, _ = layer_from_oracle(W)
    for B in (17, 33, 48, 64, 100, 128, 200, 256, 300, 600):
        _check_linear(tl, W, B, B, "gemm")
    _status_ok()


@pytest.mark.parametrize("Ms,N,regime", [((256, 64, 64), 1024, "mixed"), ((512, 128), 512, "heavy"),
                                         ((16, 16, 16, 16), 64, "mixed"), ((1024, 256, 256), 4096, "llm"),
                                         ((768, 768), 2048, "each")])
def test_gemv_list_matches_fp64(Ms, N, regime):
    """one launch over a list of matrices that share the activations (q / k / v, gate / up as separate trees): every
    member's fp32 accumulators against the oracle's fp64 product, BF16 == rounded accumulator, one-hot read-back of
    escape columns, reruns identical, exchange slots left as they were found"""
    from statetree_b200 import ops
    from statetree_b200.linear import forward_list
    E = ops.ext()
    Ws = [G.weights(M, N, 11 * i + M + N, regime) for i, M in enumerate(Ms)]
    made = [layer_from_oracle(W) for W in Ws]
    tls, encs = [m[0] for m in made], [m[1] for m in made]
    tabs = []
    for tl in tls:
        eo, el, eb = tl.tables()
        tabs.append((tl.tree, eo, eb, el))
    torch.cuda.synchronize()
    for B in (1, 3, 8, 12, 16, 27, 32):
        rs = np.random.RandomState(B)
        X = G.to_bf16_bits(rs.standard_normal((B, N)))
        x = bits_to_torch(X, DEV)
        ys = [torch.empty(B, M, dtype=torch.bfloat16, device=DEV) for M in Ms]
        yfs = [torch.empty(B, M, dtype=torch.float32, device=DEV) for M in Ms]
        nbytes = E.gemv_list_workspace_bytes(list(Ms), N, B)
        ws = torch.full((max(nbytes // 4, 1),), -1, dtype=torch.int32, device=DEV)
        args = E.gemv_list_args(tabs, ys, yfs)
        E.gemv_list(args, x, ws.view(torch.float32))
        torch.cuda.synchronize()
        assert bool((ws == -1).all()), (Ms, B, "exchange slots not restored")
        for W, y, yf in zip(Ws, ys, yfs):
            ref = oracle.linear_f64(W, X)
            assert rel_fro(yf.cpu().numpy(), ref) < TOL, (Ms, N, B)
            assert torch.equal(y, yf.to(torch.bfloat16))
        again = [torch.empty_like(y) for y in ys]
        E.gemv_list(E.gemv_list_args(tabs, again), x, ws.view(torch.float32))
        for y, z in zip(ys, again):
            assert torch.equal(y, z), (Ms, B, "nondeterministic")
    if all(M % 128 == 0 for M in Ms):                      # the same list through the tcgen05 GEMM
        from statetree_b200.linear import _state
        for B in (13, 64, 100, 256, 300):
            X = G.to_bf16_bits(np.random.RandomState(B).standard_normal((B, N)))
            x = bits_to_torch(X, DEV)
            ys = [torch.empty(B, M, dtype=torch.bfloat16, device=DEV) for M in Ms]
            yfs = [torch.empty(B, M, dtype=torch.float32, device=DEV) for M in Ms]
            cnt = _state(torch.device(DEV)).get_cnt((sum(Ms) // 128) * ((B + 255) // 256))
            E.gemm_list(E.gemv_list_args(tabs, ys, yfs), x, cnt)
            torch.cuda.synchronize()
            for W, y, yf in zip(Ws, ys, yfs):
                assert rel_fro(yf.cpu().numpy(), oracle.linear_f64(W, X)) < TOL, (Ms, N, B)
                assert torch.equal(y, yf.to(torch.bfloat16))
            assert int(cnt.abs().sum()) == 0
    # module-level helper (one launch for the list at any batch where the shapes allow) and exact read-back
    for B in (1, 8, 40):
        cols = sorted(set(np.concatenate([e["esc_cols"] for e in encs]).tolist()))[:24] + [0, N - 1]
        x = torch.zeros(B, N, dtype=torch.bfloat16, device=DEV)
        for b in range(B):
            x[b, cols[b % len(cols)]] = 1.0
        for W, y in zip(Ws, forward_list(tls, x)):
            want = bits_to_torch(np.stack([W[:, cols[b % len(cols)]] for b in range(B)]), DEV)
            assert torch.equal(y, want), (Ms, B)
    with pytest.raises(RuntimeError, match="1 to 4"):
        E.gemv_list(E.gemv_list_args(tabs * 5, [ys[0]] * (5 * len(tabs))), x[:1].contiguous(), ws.view(torch.float32))
    _status_ok()


def _one_hot_check(tl, W, cols, B):
    N = W.shape[1]
    x = torch.zeros(B, N, dtype=torch.bfloat16, device=DEV)
    for b in range(B):
        x[b, cols[b % len(cols)]] = 1.0
    y = tl(x)
    want = bits_to_torch(np.stack([W[:, cols[b % len(cols)]] for b in range(B)]), DEV)
    assert torch.equal(y, want), (W.shape, B, (y.float() - want.float()).abs().max().item())


@pytest.mark.parametrize("regime", ["mixed", "heavy", "each"])
def test_one_hot_reads_columns_back_exactly(regime):
    M, N = 256, 1024
    W = G.weights(M, N, 3, regime)
    tl, enc = layer_from_oracle(W)
    esc_cols = sorted(set(enc["esc_cols"].tolist()))
    cols = (esc_cols[:40] + list(range(0, N, 37)))[:64]                    # columns that hold escapes first
    for B in (1, 5, 8, 16, 32, 40, 64, 130):
        _one_hot_check(tl, W, cols, B)
    _status_ok()


def test_argument_errors_raise():
    from statetree_b200 import ops
    W = G.weights(64, 128, 0, "mixed")
    tl, _ = layer_from_oracle(W)
    eo, el, eb = tl.tables()
    x = torch.zeros(40, 128, dtype=torch.bfloat16, device=DEV)
    y = torch.empty(40, 64, dtype=torch.bfloat16, device=DEV)
    ws = torch.empty(16, dtype=torch.float32, device=DEV)
    cnt = torch.zeros(16, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="batch"):
        ops.ext().gemv(tl.tree, eo, eb, el, x, y, ws, cnt)
    with pytest.raises(RuntimeError, match="128"):
        ops.ext().gemm(tl.tree, eo, el, x, y, ws, cnt)                    # M = 64 is not a multiple of 128


def test_benchmark_shape_roundtrip_and_properties():
    """full-size 4096 x 4096 (the benchmark's q/o projection): lossless round trip on the GPU, one-hot read-back,
    linearity y(x1 + x2) == y(x1) + y(x2) for one-hot pairs, fp32 accumulators against torch fp64 on the GPU"""
    from statetree_b200 import TreeLinear
    W = G.weights(4096, 4096, 0, "llm")
    Wt = bits_to_torch(W, DEV)
    tl = TreeLinear.from_weight(Wt, verify=True)
    assert 0 < tl.esc_rows.numel() < 0.001 * W.size
    assert abs(tl.bits_per_weight - 12.125) < 0.05
    cols = list(range(0, 4096, 101))
    _one_hot_check(tl, W, cols, 8)
    _one_hot_check(tl, W, cols, 64)
    for B in (1, 8, 64, 256):
        x = torch.randn(B, 4096, device=DEV, generator=torch.Generator(DEV).manual_seed(B)).to(torch.bfloat16)
        yf = torch.empty(B, 4096, dtype=torch.float32, device=DEV)
        y = tl._forward(x, yf)
        ref = x.double() @ Wt.double().t()
        err = float((yf.double() - ref).norm() / ref.norm())
        assert err < TOL, (B, err)
        assert torch.equal(y, yf.to(torch.bfloat16))
    _status_ok()


@pytest.mark.gpu
def test_gemv_swiglu_matches_gemv_then_silu_mul():
    """the SwiGLU epilogue on a tile-interleaved gate/up tree against the plain product followed by st_silu_mul.  Both
    round at the same points; the two launches cut the matrix differently (whole tile pairs per CTA against equal unit
    ranges), so their fp32 sums differ in the last bits and a few BF16 outputs land on the neighbouring value."""
    import torch
    import statetree_b200 as S
    from statetree_b200.linear import interleave_gate_up
    from statetree_b200.ops import ext, lib
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(21)
    I, N = 12288, 4096
    g = (torch.randn(I, N, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    u = (torch.randn(I, N, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    g[:, 7] *= 8
    plain = S.TreeLinear.from_weight(torch.cat([g, u]), verify=False)
    inter = S.TreeLinear.from_weight(interleave_gate_up(g, u), verify=False)
    for B in (1, 3, 8):
        assert lib().st_gemv_swiglu_supported(2 * I, N, B) == 1
        x = torch.randn(B, N, device=dev, generator=gen).to(torch.bfloat16)
        y = plain(x)
        want = torch.empty(B, I, dtype=torch.bfloat16, device=dev)
        ext().silu_mul(y, want)
        got = inter.swiglu(x)
        assert torch.equal(inter.swiglu(x), got), B                                    # deterministic
        diff = (got.float() - want.float()).abs()
        assert float((diff > 0).float().mean()) < 0.02, B
        assert bool((diff <= want.float().abs() * 2.0 ** -5 + want.float().abs().max() * 2.0 ** -10).all()), B   # a few BF16 steps
    assert lib().st_gemv_swiglu_supported(2 * 48, 64, 1) in (0, 1)      # small shapes: answered, never a crash
    from statetree_b200 import ops
    assert ops.device_status() == 0


def test_workspace_growth_keeps_captured_graphs_valid():
    """a CUDA graph captured at one shape keeps replaying correctly after a much larger shape has made the shared
    workspace grow: buffers that were handed out are retired, never freed"""
    from statetree_b200.linear import _state
    W = G.weights(512, 1024, 21, "mixed")
    tl, _ = layer_from_oracle(W)
    x = bits_to_torch(G.to_bf16_bits(np.random.RandomState(1).standard_normal((3, 1024))), DEV)
    want = tl(x).clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        st = _state(torch.device(DEV))
        y = tl(x)
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        y = tl(x)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        before = st.ws.data_ptr()
        big, _ = layer_from_oracle(G.weights(4096, 8192, 22, "llm"))
        xb = bits_to_torch(G.to_bf16_bits(np.random.RandomState(2).standard_normal((12, 8192))), DEV)
        st.get_ws(st.ws.numel() * 4 + (64 << 20))             # force the workspace of this stream to grow
        assert st.ws.data_ptr() != before and len(st._retired) >= 1
        big(xb)
        filler = [torch.full((1 << 20,), 0.5, device=DEV) for _ in range(8)]   # whatever the allocator hands out next
    side.synchronize()
    for _ in range(3):
        y.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    del filler
    _status_ok()


@pytest.mark.parametrize("M,N,B,act", [(512, 1024, 1, False), (1024, 4096, 3, False), (2048, 2048, 8, False),
                                       (24576, 4096, 1, True), (12288, 2048, 4, True)])
def test_gemv_prenorm_equals_add_rmsnorm_then_gemv(M, N, B, act):
    """the GEMV that forms RMSNorm(x + delta) * w itself against the two-launch sequence it replaces: the new residual
    stream bit for bit, the product within a BF16 step (the two sum the squares in different orders)"""
    from statetree_b200 import ops, TreeLinear
    from statetree_b200.linear import _state, interleave_gate_up
    E = ops.ext()
    gen = torch.Generator(device=DEV).manual_seed(M + N + B)
    W = (torch.randn(M, N, device=DEV, generator=gen) * 0.05).to(torch.bfloat16)
    if act:
        W = interleave_gate_up(W[:M // 2].contiguous(), W[M // 2:].contiguous())
    if not E.gemv_prenorm_supported(M, N, B, act):
        pytest.skip("shape not taken by the fused epilogue on this GPU")
    tl = TreeLinear.from_weight(W, verify=False)
    eo, el, eb = tl.tables()
    torch.cuda.synchronize()
    x = torch.randn(B, N, device=DEV, generator=gen).to(torch.bfloat16)
    d = torch.randn(B, N, device=DEV, generator=gen).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(N, device=DEV, generator=gen)).to(torch.bfloat16)
    st = _state(torch.device(DEV))
    ws = st.get_ws(E.gemv_workspace_bytes(M, N, B))
    for delta in (d, None):
        x_ref, h = x.clone(), torch.empty_like(x)
        E.add_rmsnorm(x_ref, delta, nw, h, 1e-6)
        want = tl.swiglu(h) if act else tl(h)
        x_out = torch.zeros_like(x)
        got = torch.empty(B, M // 2 if act else M, dtype=torch.bfloat16, device=DEV)
        E.gemv_prenorm(tl.tree, eo, eb, el, x, delta, nw, 1e-6, x_out, got, ws, act)
        torch.cuda.synchronize()
        assert torch.equal(x_out, x_ref)
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2 ** -6 * want.float().abs().max().item() + 1e-6, (M, N, B, act, err)
        again = torch.empty_like(got)
        E.gemv_prenorm(tl.tree, eo, eb, el, x, delta, nw, 1e-6, x_out, again, ws, act)
        assert torch.equal(got, again)
    _status_ok()


def test_prefill_batches_decode_once_and_use_the_dense_product():
    """more than PREFILL_MIN activation rows: the layer is decoded into a BF16 scratch matrix and cuBLAS multiplies by
    it (the reference's path above 1024 rows); the layer linked as next is decoded on a side stream meanwhile.  Same
    bits as the product with the dequantized weight, within BF16 rounding of the fp64 product, whatever the order the
    layers are called in."""
    import pickle
    import weakref
    import statetree_b200.linear as L
    shapes = [(512, 1024), (1024, 512), (256, 1024)]
    Ws = [G.weights(M, N, 31 * i + M, "mixed") for i, (M, N) in enumerate(shapes)]
    tls = [layer_from_oracle(W)[0] for W in Ws]
    for a, b in zip(tls, tls[1:] + tls[:1]):
        a.__dict__["_next"] = weakref.ref(b)
    B = L.PREFILL_MIN + 300
    stage = L._state(torch.device(DEV)).dense_stage()

    def check(i, seed):
        W, tl = Ws[i], tls[i]
        X = G.to_bf16_bits(np.random.RandomState(seed).standard_normal((B, W.shape[1])))
        x = bits_to_torch(X, DEV)
        y = tl(x)
        assert torch.equal(y, torch.matmul(x, tl.dequantize().t())), (i, "not the dense product")
        assert rel_fro(y.float().cpu().numpy(), oracle.linear_f64(W, X)) < 5e-3, i

    check(0, 1)
    assert stage.holds[1 - stage.holds.index(stage._ident(tls[0]))] == stage._ident(tls[1])   # next layer prefetched
    check(1, 2)                                             # served from the prefetched matrix
    check(2, 3)
    check(0, 4)                                             # wrapped around
    check(2, 5)                                             # not the predicted layer: decoded on demand
    check(2, 6)
    check(1, 7)
    torch.cuda.synchronize()
    y_small = tls[0](bits_to_torch(G.to_bf16_bits(np.random.RandomState(9).standard_normal((64, 1024))), DEV))
    assert y_small.shape == (64, 512)                       # smaller batches still take the tree kernels
    tls[1].allow_dec = False                                # as for a vocabulary-sized table: tree kernels at any batch
    xb = bits_to_torch(G.to_bf16_bits(np.random.RandomState(11).standard_normal((B, 512))), DEV)
    yk = tls[1](xb)
    parts = torch.cat([tls[1](xb[i:i + 512]) for i in range(0, B, 512)])
    assert rel_fro(yk.float().cpu().numpy(), parts.float().cpu().numpy()) < 5e-3
    clone = pickle.loads(pickle.dumps(tls[0].cpu()))        # the link to the next layer does not travel
    assert clone.__dict__["_next"] is None
    _status_ok()


def test_layer_prepare_then_graph_capture():
    """TreeLinear.prepare builds the side tables and sizes the workspaces, so the first call may be a captured one"""
    W = G.weights(256, 512, 5, "mixed")
    tl, _ = layer_from_oracle(W)
    assert tl._tables is None
    tl.prepare([1, 64]).set_handle("blk0.q_proj")
    assert tl._tables is not None
    import statetree_b200.linear as L
    assert L._BY_HANDLE["blk0.q_proj"] is tl
    for B in (1, 64):
        x = bits_to_torch(G.to_bf16_bits(np.random.RandomState(B).standard_normal((B, 512))), DEV)
        y = torch.empty(B, 256, dtype=torch.bfloat16, device=DEV)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            L._state(torch.device(DEV))                     # (workspaces are per stream: size this stream's too)
            tl.prepare([B])
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                tl._run(x, y)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, tl(x)), B
    _status_ok()
