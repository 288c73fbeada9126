"""Generates the golden fixtures of this folder by importing the REFERENCE implementation (statetree/format.py of the
upstream project) and running it on seeded inputs.  Run once, in a container that holds the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The fixtures (small .npz files and a table of SHA-256 digests for the larger cases) are committed; tests never import
the reference.
"""
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import gen_inputs as G  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def ref_encode(F, bits):
    W = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
    enc = F.encode(W)
    back = F.decode_reference(enc["tree"], enc["esc_rows"], enc["esc_cols"], enc["esc_bits"])
    assert torch.equal(back.view(torch.int16), W.view(torch.int16))
    return {k: v.numpy() for k, v in enc.items()}


def main(ref_root):
    sys.path.insert(0, ref_root)
    from statetree import format as F

    # 1. small matrices stored whole (inputs and reference outputs)
    small = {}
    for name, (M, N, seed, regime) in {"mixed": (128, 256, 1, "mixed"), "heavy": (32, 128, 2, "heavy"),
                                       "each": (32, 192, 3, "each"), "llm": (64, 128, 4, "llm")}.items():
        bits = G.weights(M, N, seed, regime)
        enc = ref_encode(F, bits)
        small[f"{name}_W"] = bits
        for k, v in enc.items():
            small[f"{name}_{k}"] = v
        eo, el = F.escape_lists(M, N, enc_t(enc, "esc_rows"), enc_t(enc, "esc_cols"), enc_t(enc, "esc_bits"))
        small[f"{name}_eo"] = eo.numpy()
        small[f"{name}_el"] = el.numpy()
    np.savez_compressed(os.path.join(HERE, "weights_small.npz"), **small)

    # 2. larger matrices: digests only (inputs are regenerated from the seed by gen_inputs.weights)
    digests = {}
    for M, N, seed, regime in ((256, 512, 0, "mixed"), (512, 1024, 1, "mixed"), (256, 2048, 5, "heavy"),
                               (1024, 512, 6, "each"), (1024, 1024, 0, "llm"), (512, 768, 7, "llm")):
        bits = G.weights(M, N, seed, regime)
        enc = ref_encode(F, bits)
        esc = (enc_t(enc, "esc_rows"), enc_t(enc, "esc_cols"), enc_t(enc, "esc_bits"))
        side = {}                                        # the reference's side tables (format.py:141-216)
        for tag, out in (("lists", F.escape_lists(M, N, *esc)), ("chunks", F.escape_chunks(M, N, *esc)),
                         ("blocks1", F.escape_blocks(M, N, 1, *esc)), ("blocks2", F.escape_blocks(M, N, 2, *esc))):
            side[tag] = [sha(t.numpy()) for t in out]
        leaves_v1 = F._v1(enc_t(enc, "tree")[..., :1024].to(torch.int32)).to(torch.uint8).numpy()
        digests[f"{M}x{N}_s{seed}_{regime}"] = dict(
            M=M, N=N, seed=seed, regime=regime, n_esc=int(enc["esc_rows"].size), W=sha(bits), tree=sha(enc["tree"]),
            esc_rows=sha(enc["esc_rows"]), esc_cols=sha(enc["esc_cols"]), esc_bits=sha(enc["esc_bits"]),
            bits_per_weight=F.bits_per_weight(M, N, int(enc["esc_rows"].size)), side_tables=side,
            leaves_v1=sha(leaves_v1), PERM=list(F.PERM))
    with open(os.path.join(HERE, "weights_digests.json"), "w") as f:
        json.dump(digests, f, indent=1, sort_keys=True)

    # 3. KV records: a record is the format.py encoding of a [16 tokens, 64 dims] block (token = row); its first 11
    #    escapes in (row, col) order fill the in-record slots as bits << 16 | row << 6 | col
    K, V = G.kv_tokens(48, 2, seed=11, tiny=0.03)
    Kc, Vc = G.kv_tokens(32, 2, seed=12, tiny=0.0, channel_scale=True)
    kv = {}
    for name, (k, v) in {"tiny": (K, V), "chan": (Kc, Vc)}.items():
        n, H, _ = k.shape
        recs, counts, slots = [], [], []
        for arr in (k, v):
            for p in range(n // 16):
                for h in range(H):
                    for half in range(2):
                        blk = np.ascontiguousarray(arr[p * 16:(p + 1) * 16, h, half * 64:(half + 1) * 64])
                        enc = ref_encode(F, blk)
                        recs.append(enc["tree"].reshape(1552))
                        ent = (enc["esc_bits"].astype(np.int64) & 0xFFFF) << 16 | enc["esc_rows"].astype(np.int64) << 6 \
                            | enc["esc_cols"].astype(np.int64)
                        counts.append(ent.size)
                        s = np.zeros(11, dtype=np.uint32)
                        s[:min(11, ent.size)] = ent[:11].astype(np.uint32)
                        slots.append(s)
        kv[f"{name}_K"], kv[f"{name}_V"] = k, v
        kv[f"{name}_records"] = np.stack(recs)            # order: (K then V, page, head, half)
        kv[f"{name}_counts"] = np.array(counts, dtype=np.int32)
        kv[f"{name}_slots"] = np.stack(slots)
    np.savez_compressed(os.path.join(HERE, "kv_records.npz"), **kv)
    print("wrote fixtures to", HERE)


def enc_t(enc, k):
    return torch.from_numpy(enc[k])


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference-checkout")
    main(sys.argv[1])
