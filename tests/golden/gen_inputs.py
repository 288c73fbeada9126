"""Seeded synthetic inputs shared by the golden-fixture generator and the tests (pure numpy: the legacy RandomState
stream is frozen, so the same seed gives the same bits everywhere).  BF16 values are uint16 bit patterns."""
import numpy as np


def to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def weights(M, N, seed=0, regime="mixed"):
    """BF16 weight matrices in the escape regimes the reference's kernel tests exercise:
    'llm'    N(0, 0.02) with 1% of the columns scaled x8 (the benchmark distribution, ~0.017% escapes)
    'mixed'  N(0, 0.02) + an exact zero, a run of 1e-9, an outlier 3.0, a dense zero cluster
    'heavy'  20% of the weights scaled by 1e-6 (hundreds of escapes per record)
    'each'   exactly one escape in every record"""
    rs = np.random.RandomState(seed)
    W = (rs.standard_normal((M, N)) * 0.02).astype(np.float32)
    if regime == "llm":
        cols = rs.permutation(N)[:max(1, N // 100)]
        W[:, cols] *= 8.0
    elif regime == "mixed":
        W[3, 5] = 0.0
        W[min(17, M - 1), 70:90] = 1e-9
        W[min(40, M - 1), min(128, N - 1)] = 3.0
        W[min(100, M - 4):min(104, M), 0:64:2] = 0.0
    elif regime == "heavy":
        W[rs.random_sample((M, N)) < 0.2] *= 1e-6
    elif regime == "each":
        W = np.where(np.abs(W) < 1e-4, np.float32(1e-3), W)
        for t in range(M // 16):
            for g in range(N // 64):
                W[t * 16 + rs.randint(16), g * 64 + rs.randint(64)] = 0.0
    else:
        raise ValueError(regime)
    return to_bf16_bits(W)


def kv_tokens(n, H, seed=0, tiny=0.02, channel_scale=False):
    """K, V [n, H, 128] bf16 bits.  tiny: fraction of values scaled by 2^-30 (escapes), plus 1% exact zeros, as the
    reference's page tests; channel_scale: K = N(0,1) x LogNormal(0,1) per channel (the benchmark distribution)."""
    rs = np.random.RandomState(seed)
    x = rs.standard_normal((2, n, H, 128)).astype(np.float32)
    if channel_scale:
        x[0] *= np.exp(rs.standard_normal((H, 128))).astype(np.float32)
    if tiny > 0:
        x = np.where(rs.random_sample(x.shape) < tiny, x * np.float32(2.0 ** -30), x)
        x = np.where(rs.random_sample(x.shape) < 0.01, np.float32(0.0), x)
    b = to_bf16_bits(x)
    return b[0], b[1]
