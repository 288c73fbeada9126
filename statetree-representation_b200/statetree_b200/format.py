"""Lossless state-tree format for BF16 matrices: same API and byte-identical output as the reference's
statetree/format.py (encode 66-83, decode_reference 101-121, escape_count 87-97, bits_per_weight 219-221).

A BF16 value is sign | 8-bit exponent | 7-bit mantissa.  Rows are cut into groups of 64; per group the largest
exponent E is kept once (node), every value keeps a 4-bit state D = E - exponent and an 8-bit leaf
(mantissa << 1 | sign of its pair partner).  D = 15 marks an escape (exponent more than 14 below E) whose exact bits
go to a side list.  One 1552-byte record holds a 16-row x 64-column block in mma.m16n8k16 A-fragment order.

This implementation places bytes through three lookup tables (leaf / state / node position of element (r, c) of a
record) instead of the reference's chain of reshapes; the tables are the closed form also used by the KV kernels
(statetree/csrc/kvcache.cu:31-38).  It runs on the tensor's device (CPU works and is what the tests pin against the
golden fixtures).  The side tables the kernels of this package read are built by escape_tables().
"""
import torch

RECORD_BYTES = 1552
LEAF_FORMAT = 2                      # leaf byte = mantissa << 1 | partner's sign; format 1 was sign << 7 | mantissa
# column (0..63) that thread-in-quad t of a lane holds at byte position p of its 16 leaf bytes of one record half-row:
# k-step p // 4, upper half of the k-step (p // 2) % 2, element of the pair p % 2 (the reference's format.PERM)
PERM = [16 * (p >> 2) + 8 * ((p >> 1) & 1) + 2 * t + (p & 1) for t in range(4) for p in range(16)]
_LUT = {}


def _luts(device):
    """(leaf_pos [16, 64], state_pos [8, 64], node_pos [16]) int64 byte offsets inside a record"""
    key = str(device)
    if key not in _LUT:
        r = torch.arange(16).view(16, 1)
        c = torch.arange(64).view(1, 64)
        pair = c // 2
        s, t, hi = pair >> 3, pair & 3, (pair >> 2) & 1
        leaf = (s >> 1) * 512 + ((r & 7) * 4 + t) * 16 + ((s & 1) * 2 + (r >> 3)) * 4 + 2 * hi + (c & 1)
        state = 1024 + ((r[:8] & 7) * 4 + t) * 16 + s * 4 + 2 * hi + (c & 1)
        node = 1536 + 2 * (torch.arange(16) & 7) + (torch.arange(16) >> 3)
        _LUT[key] = tuple(x.to(device) for x in (leaf, state, node))
    return _LUT[key]


def _fields(W):
    b = W.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    return b, (b >> 15) & 1, (b >> 7) & 0xFF, b & 0x7F


def _encode_chunk(W):
    """W [m, N] bf16 (m % 16 == 0) -> records uint8 [m/16, N/64, 1552], escape (row, col, bits)"""
    m, N = W.shape
    T, NG = m // 16, N // 64
    leaf_pos, state_pos, node_pos = _luts(W.device)
    bits, sign, expo, mant = _fields(W)
    eg = expo.view(m, NG, 64)
    E = eg.amax(-1)                                            # [m, NG]
    D = E.unsqueeze(-1) - eg
    esc = D > 14
    keep = ~esc
    mant_k = mant.view(m, NG, 64) * keep
    sign_k = sign.view(m, NG, 64) * keep
    partner = sign_k.view(m, NG, 32, 2).flip(-1).reshape(m, NG, 64)
    leaf = (mant_k << 1) | partner
    Dq = torch.where(esc, torch.full_like(D, 15), D)
    # [m, NG, 64] -> [T, NG, 16, 64]
    leaf = leaf.view(T, 16, NG, 64).permute(0, 2, 1, 3)
    Dq = Dq.view(T, 16, NG, 64).permute(0, 2, 1, 3)
    rec = torch.zeros(T, NG, RECORD_BYTES, dtype=torch.uint8, device=W.device)
    rec[:, :, leaf_pos.reshape(-1)] = leaf.reshape(T, NG, 1024).to(torch.uint8)
    nib = Dq[:, :, :8] | (Dq[:, :, 8:] << 4)                   # rows g and g + 8 share a byte
    rec[:, :, state_pos.reshape(-1)] = nib.reshape(T, NG, 512).to(torch.uint8)
    rec[:, :, node_pos] = E.view(T, 16, NG).permute(0, 2, 1).to(torch.uint8)
    er, ec = esc.view(m, N).nonzero(as_tuple=True)
    return rec, er, ec, W.contiguous().view(torch.int16)[er, ec]


@torch.no_grad()
def encode(W, chunk_rows=4096):
    """W [M, N] bf16 (M % 16 == 0, N % 64 == 0) -> dict(tree uint8 [M/16, N/64, 1552], esc_rows / esc_cols int32,
    esc_bits int16), escapes in (row, col) order.  Runs on W's device in row chunks."""
    assert W.dim() == 2 and W.dtype == torch.bfloat16, "encode expects a 2-D bf16 matrix"
    M, N = W.shape
    assert M % 16 == 0 and N % 64 == 0, f"shape {tuple(W.shape)}: rows must be a multiple of 16, cols of 64"
    chunk_rows = max(16, chunk_rows // 16 * 16)
    tree = torch.empty(M // 16, N // 64, RECORD_BYTES, dtype=torch.uint8, device=W.device)
    rows, cols, bits = [], [], []
    for r0 in range(0, M, chunk_rows):
        rec, er, ec, eb = _encode_chunk(W[r0:r0 + chunk_rows])
        tree[r0 // 16:r0 // 16 + rec.shape[0]] = rec
        del rec
        rows.append((er + r0).to(torch.int32))
        cols.append(ec.to(torch.int32))
        bits.append(eb)
    return dict(tree=tree, esc_rows=torch.cat(rows), esc_cols=torch.cat(cols), esc_bits=torch.cat(bits))


@torch.no_grad()
def escape_count(W, chunk_rows=8192):
    """how many values of W [..., N] the tree cannot hold (the escapes encode() would list)"""
    assert W.dtype == torch.bfloat16 and W.shape[-1] % 64 == 0
    W2 = W.reshape(-1, W.shape[-1])
    n = 0
    for r0 in range(0, W2.shape[0], chunk_rows):
        e = (W2[r0:r0 + chunk_rows].contiguous().view(torch.int16).to(torch.int32) >> 7) & 0xFF
        e = e.view(e.shape[0], -1, 64)
        n += int(((e.amax(-1, keepdim=True) - e) > 14).sum())
    return n


@torch.no_grad()
def decode_reference(tree, esc_rows, esc_cols, esc_bits):
    """Pure-torch decode (slow; the CUDA `dec` kernel is the fast path): the exact bf16 matrix."""
    T, NG, _ = tree.shape
    M, N = T * 16, NG * 64
    leaf_pos, state_pos, node_pos = _luts(tree.device)
    rec = tree.to(torch.int32)
    leaf = rec[:, :, leaf_pos.reshape(-1)].view(T, NG, 16, 64)
    nib = rec[:, :, state_pos.reshape(-1)].view(T, NG, 8, 64)
    D = torch.cat([nib & 15, nib >> 4], 2)                     # rows 0..7 low nibble, 8..15 high nibble
    E = rec[:, :, node_pos].view(T, NG, 16, 1)
    sign = (leaf.view(T, NG, 16, 32, 2).flip(-1).reshape(T, NG, 16, 64)) & 1
    ex = (E - D).clamp(min=0)
    bits = (sign << 15) | (ex << 7) | (leaf >> 1)
    bits = bits.permute(0, 2, 1, 3).reshape(M, N)
    bits = torch.where(bits >= 32768, bits - 65536, bits).to(torch.int16)
    if esc_rows.numel():
        bits[esc_rows.long(), esc_cols.long()] = esc_bits
    return bits.view(torch.bfloat16)


@torch.no_grad()
def leaves_v1_to_v2(tree):
    """records written with leaf format 1 (sign << 7 | mantissa, checkpoints of version < 3) -> leaf format 2; the
    two bytes of a BF16 pair sit next to each other, states and nodes are untouched
    (reference: statetree/format.py:36-40)"""
    out = tree.clone()
    old = out[..., :1024].to(torch.int32)
    pairs = old.reshape(*old.shape[:-1], 512, 2)
    new = ((pairs & 0x7F) << 1) | (pairs.flip(-1) >> 7)
    out[..., :1024] = new.reshape(old.shape).to(torch.uint8)
    return out


@torch.no_grad()
def leaves_v2_to_v1(tree):
    """inverse of leaves_v1_to_v2 (used to write version-2 files for the migration test)"""
    out = tree.clone()
    new = out[..., :1024].to(torch.int32)
    pairs = new.reshape(*new.shape[:-1], 512, 2)
    old = ((pairs.flip(-1) & 1) << 7) | (pairs >> 1)
    out[..., :1024] = old.reshape(new.shape).to(torch.uint8)
    return out


def _u32(x):
    """int64 values in [0, 2^32) -> the same bit patterns as int32"""
    return torch.where(x >= 2 ** 31, x - 2 ** 32, x).to(torch.int32).contiguous()


def units_per_tile(N):
    """units (up to 8 consecutive records of a 16-row tile) per tile: the work unit of the GEMV kernel"""
    return (N // 64 + 7) // 8


@torch.no_grad()
def escape_tables(M, N, esc_rows, esc_cols, esc_bits):
    """Side tables the kernels read (built once per matrix, on the escape lists' device):
      eo int32 [records + 1]   offsets of each record's entries in el (records in memory order: tile * N/64 + group)
      el int32 [max(n, 1)]     entries bits << 16 | (record % 8) << 10 | row << 6 | col, sorted by record
      eb int32 [units, 16]     per GEMV unit: count | (mask of records with escapes) << 16, offset into el, the first
                               14 entries inline
    They play the role of the reference's escape_lists / escape_chunks (statetree/format.py:141-154, 189-216)."""
    dev = esc_rows.device
    NG = N // 64
    nrec = (M // 16) * NG
    cpt = units_per_tile(N)
    nunit = (M // 16) * cpt
    rows, cols = esc_rows.long(), esc_cols.long()
    bits = esc_bits.to(torch.int64) & 0xFFFF
    tile, r, G, c = rows // 16, rows % 16, cols // 64, cols % 64
    rec = tile * NG + G
    ent = (bits << 16) | ((G & 7) << 10) | (r << 6) | c
    order = torch.argsort(rec, stable=True)
    ent_s = ent[order]
    eo = torch.zeros(nrec + 1, dtype=torch.int64, device=dev)
    if rec.numel():
        eo[1:] = torch.bincount(rec, minlength=nrec).cumsum(0)
    eb = torch.zeros(nunit, 16, dtype=torch.int64, device=dev)
    first_rec = (torch.arange(M // 16, device=dev).view(-1, 1) * NG + torch.arange(cpt, device=dev).view(1, -1) * 8)
    eb[:, 1] = eo[first_rec.reshape(-1)]
    if rec.numel():
        unit_s = (tile * cpt + G // 8)[order]
        eb[:, 0] = torch.bincount(unit_s, minlength=nunit)
        rec_bit = torch.zeros(nunit * 8, dtype=torch.int64, device=dev)
        rec_bit[unit_s * 8 + (ent_s >> 10 & 7)] = 1                       # which records of the unit have escapes
        eb[:, 0] |= (rec_bit.view(nunit, 8) << torch.arange(16, 24, device=dev)).sum(1)
        pos = torch.arange(ent_s.numel(), device=dev) - eb[unit_s, 1]
        keep = pos < 14
        eb[unit_s[keep], 2 + pos[keep]] = ent_s[keep]
    el = _u32(ent_s) if ent_s.numel() else torch.zeros(1, dtype=torch.int32, device=dev)
    return eo.to(torch.int32).contiguous(), el, _u32(eb.view(-1)).view(nunit, 16)


# ---- the reference's side-table builders (statetree/format.py:141-216), kept for callers of its format module.  The
# kernels of this package read escape_tables() above; these produce the reference's tables bit for bit.
def _fragment_entry(esc_rows, esc_cols, esc_bits):
    """per escape: (tile, column group, k-step, entry) with entry = bits << 16 | lane << 5 | k-step << 3 | reg << 1 |
    half, i.e. where the value sits in the mma.m16n8k16 A fragment of its record"""
    r, c = esc_rows.long(), esc_cols.long()
    row, col = r % 16, c % 64
    kstep, k = col // 16, col % 16
    lane = (row % 8) * 4 + (k % 8) // 2
    reg = row // 8 + 2 * (k // 8)
    ent = ((esc_bits.to(torch.int64) & 0xFFFF) << 16) | (lane << 5) | (kstep << 3) | (reg << 1) | (k % 2)
    return r // 16, c // 64, kstep, ent


def _unit_blocks(unit, slot, kstep, ent, n_units):
    """64-byte blocks per unit of 8 records: words 0-1 = bit (slot * 4 + k-step) per escape, word 2 = count, words
    3..15 = the first 13 entries (entry | slot << 10); plus offsets per unit and the full sorted list"""
    dev = unit.device
    ent = ent | (slot << 10)
    order = torch.argsort(unit, stable=True)
    u_s, e_s = unit[order], ent[order]
    count = torch.bincount(unit, minlength=n_units) if unit.numel() else torch.zeros(n_units, dtype=torch.int64, device=dev)
    offs = torch.zeros(n_units + 1, dtype=torch.int64, device=dev)
    offs[1:] = count.cumsum(0)
    blocks = torch.zeros(n_units, 16, dtype=torch.int64, device=dev)
    blocks[:, 2] = count
    if unit.numel():
        bit = slot * 4 + kstep
        flags = torch.zeros(n_units, 64, dtype=torch.int64, device=dev)
        flags[unit, bit] = 1
        weights = torch.ones(32, dtype=torch.int64, device=dev) << torch.arange(32, device=dev)
        blocks[:, 0] = (flags[:, :32] * weights).sum(1)
        blocks[:, 1] = (flags[:, 32:] * weights).sum(1)
        rank = torch.arange(u_s.numel(), device=dev) - offs[u_s]
        inline = rank < 13
        blocks[u_s[inline], 3 + rank[inline]] = e_s[inline]
    full = _u32(e_s) if e_s.numel() else torch.zeros(1, dtype=torch.int32, device=dev)
    return _u32(blocks.view(-1)), offs.to(torch.int32).contiguous(), full


@torch.no_grad()
def escape_lists(M, N, esc_rows, esc_cols, esc_bits):
    """(EO int32 [records + 1], EL int32): per record (tile * N/64 + group) its fragment entries"""
    NG, nrec = N // 64, (M // 16) * (N // 64)
    tile, grp, _, ent = _fragment_entry(esc_rows, esc_cols, esc_bits)
    rec = tile * NG + grp
    eo = torch.zeros(nrec + 1, dtype=torch.int64, device=esc_rows.device)
    if rec.numel():
        eo[1:] = torch.bincount(rec, minlength=nrec).cumsum(0)
    ent = ent[torch.argsort(rec, stable=True)]
    el = _u32(ent) if ent.numel() else torch.zeros(1, dtype=torch.int32, device=esc_rows.device)
    return eo.to(torch.int32).contiguous(), el


@torch.no_grad()
def escape_blocks(M, N, RT, esc_rows, esc_cols, esc_bits):
    """(EB int32 [U * 16], EOU int32 [U + 1], EALL int32) for units = (block of RT row tiles, column group)"""
    NG = N // 64
    tile, grp, kstep, ent = _fragment_entry(esc_rows, esc_cols, esc_bits)
    return _unit_blocks((tile // RT) * NG + grp, tile % RT, kstep, ent, (M // 16 // RT) * NG)


@torch.no_grad()
def escape_chunks(M, N, esc_rows, esc_cols, esc_bits):
    """the same blocks for units of 8 consecutive records in memory order"""
    NG = N // 64
    tile, grp, kstep, ent = _fragment_entry(esc_rows, esc_cols, esc_bits)
    rec = tile * NG + grp
    return _unit_blocks(rec // 8, rec % 8, kstep, ent, (M // 16) * NG // 8)


def bits_per_weight(M, N, n_esc, esc_bytes=10):
    """stored size: records + escape list (row, col: 4 B each, bits: 2 B)"""
    return ((M // 16) * (N // 64) * RECORD_BYTES * 8 + n_esc * esc_bytes * 8) / (M * N)
