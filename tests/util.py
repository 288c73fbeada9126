"""helpers shared by the tests: numpy bf16 bit patterns <-> torch tensors, oracle-encoded layers on the GPU"""
import numpy as np
import torch


def bits_to_torch(bits, device="cpu"):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16).to(device)


def torch_to_bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def rel_fro(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def layer_from_oracle(W_bits, device="cuda"):
    """TreeLinear whose buffers come from the ORACLE's encode (not from the package's own encoder)"""
    import oracle
    from statetree_b200 import TreeLinear
    enc = oracle.encode(W_bits)
    M, N = W_bits.shape
    tl = TreeLinear(N, M, device="meta", n_esc=int(enc["esc_rows"].size))
    tl._buffers["tree"] = torch.from_numpy(enc["tree"]).to(device)
    tl._buffers["esc_rows"] = torch.from_numpy(enc["esc_rows"]).to(device)
    tl._buffers["esc_cols"] = torch.from_numpy(enc["esc_cols"]).to(device)
    tl._buffers["esc_bits"] = torch.from_numpy(enc["esc_bits"]).to(device)
    tl._reset_runtime()
    return tl, enc
