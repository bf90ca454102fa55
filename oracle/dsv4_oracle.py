"""CPU oracle for the DeepSeek-V4 decode-attention path (TEST INFRASTRUCTURE ONLY).

This module restates, in numpy, the arithmetic of the reference project's
PyTorch decode path.  It is the checker the CUDA kernels are compared with; it
is never part of the shipped compute path.  Only the tests, the smoke check and
the CPU-baseline leg of the benchmark may import it.

Parity pin: `tests/golden/*.npz` hold outputs of the reference's own
`hca_decode_forward` (bench/bench/reference.py:471-546) on the seeded inputs
that `tests/golden/gen_golden.py` builds; `tests/test_oracle.py` checks every
function here against them.  Semantics the reference does not define (paged
pools, block tables, -1 padded index lists, per-128 FP32 scales, the LSE
output) are pinned only by this restatement and are marked "unpinned by the
reference" where they appear.

Reference lines each function follows are cited in its docstring as
`path:line` inside the reference project.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np

# ── entry layout (one compressed-KV cache entry) ────────────────────────
D_LATENT = 512            # FP8 e4m3 latent, also the value width d_v
D_ROPE = 64               # BF16 RoPE tail
D_QK = D_LATENT + D_ROPE  # 576
SCALE_BLOCK = 128         # one FP32 absmax scale per 128 latent elements
N_SCALES = D_LATENT // SCALE_BLOCK
SCALE_OFF = D_LATENT                      # byte offset of the 4 FP32 scales
ROPE_OFF = D_LATENT + 4 * N_SCALES        # byte offset of the 64 BF16 rope values
ENTRY_BYTES = ROPE_OFF + 2 * D_ROPE       # 656
PAGE_ENTRIES = 64
E4M3_MAX = 448.0


# ── bf16 / e4m3 scalar formats ──────────────────────────────────────────

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit pattern (uint16)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = rounded.astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def _build_e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for byte in range(256):
        s = -1.0 if byte & 0x80 else 1.0
        e = (byte >> 3) & 0xF
        m = byte & 0x7
        if e == 0xF and m == 0x7:
            v = float("nan")
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[byte] = v
    return t


E4M3_TABLE = _build_e4m3_table()
# Positive finite e4m3 magnitudes in increasing order (codes 0x00..0x7E).
_E4M3_POS = E4M3_TABLE[:0x7F].astype(np.float64)
# Midpoints between neighbours; ties go to the even code.
_E4M3_MID = (_E4M3_POS[:-1] + _E4M3_POS[1:]) / 2.0


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.ascontiguousarray(b, dtype=np.uint8)]


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 (fn variant) byte, round-to-nearest-even, saturating at
    +-448.  Same result as `x.clamp(-448, 448).to(torch.float8_e4m3fn)`, the
    conversion the reference's quantiser uses (bench/bench/decode.py:110-113)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    mag = np.minimum(np.abs(x.astype(np.float64)), E4M3_MAX)
    # code = number of midpoints strictly below mag, ties resolved to even
    code = np.searchsorted(_E4M3_MID, mag, side="left").astype(np.int64)
    tie = (code < _E4M3_MID.size) & (mag == _E4M3_MID[np.minimum(code, _E4M3_MID.size - 1)])
    # at a tie `code` is the lower neighbour; go up when the lower one is odd
    code = np.where(tie & ((code & 1) == 1), code + 1, code)
    out = code.astype(np.uint8)
    out = np.where(np.signbit(x), out | 0x80, out).astype(np.uint8)
    return out


# ── quantise / pack / unpack of cache entries ───────────────────────────

def quantize_latent(latent: np.ndarray):
    """[..., 512] float32 -> (e4m3 bytes [..., 512], FP32 scales [..., 4]).

    Follows the reference quantiser's recipe (bench/bench/decode.py:92-114:
    per-tile absmax, value/scale clamped to +-448, e4m3 cast) with the tile and
    scale type this library's cache uses: one FP32 scale = absmax/448 per 128
    elements instead of a power-of-two byte per 64.  A block of zeros gets
    scale 1 (unpinned by the reference)."""
    latent = np.ascontiguousarray(latent, dtype=np.float32)
    lead = latent.shape[:-1]
    blk = latent.reshape(*lead, N_SCALES, SCALE_BLOCK)
    absmax = np.abs(blk).max(axis=-1)
    scale = (absmax / np.float32(E4M3_MAX)).astype(np.float32)
    scale = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
    q = f32_to_e4m3((blk / scale[..., None]).astype(np.float32))
    return q.reshape(*lead, D_LATENT), scale


def pack_entries(latent: np.ndarray, rope: np.ndarray) -> np.ndarray:
    """float32 latent [..., 512] + rope [..., 64] -> uint8 [..., 656]."""
    q, scale = quantize_latent(latent)
    lead = q.shape[:-1]
    out = np.empty((*lead, ENTRY_BYTES), dtype=np.uint8)
    out[..., :D_LATENT] = q
    out[..., SCALE_OFF:ROPE_OFF] = scale.view(np.uint8).reshape(*lead, 4 * N_SCALES)
    out[..., ROPE_OFF:] = f32_to_bf16_bits(rope).view(np.uint8).reshape(*lead, 2 * D_ROPE)
    return out


def unpack_entries(entries: np.ndarray) -> np.ndarray:
    """uint8 [..., 656] -> exactly dequantised float32 rows [..., 576].

    Dequantisation is `fp8 value * scale` in float32, the exact dequant the
    reference applies before its attention math
    (bench/bench/reference.py:422-442, with this cache's FP32 scale)."""
    entries = np.ascontiguousarray(entries, dtype=np.uint8)
    lead = entries.shape[:-1]
    lat = e4m3_to_f32(entries[..., :D_LATENT]).reshape(*lead, N_SCALES, SCALE_BLOCK)
    scale = np.ascontiguousarray(entries[..., SCALE_OFF:ROPE_OFF]).view(np.float32)
    lat = (lat * scale.reshape(*lead, N_SCALES, 1)).reshape(*lead, D_LATENT)
    rope = bf16_bits_to_f32(np.ascontiguousarray(entries[..., ROPE_OFF:]).view(np.uint16))
    return np.concatenate([lat, rope.reshape(*lead, D_ROPE)], axis=-1).astype(np.float32)


# ── the attention core ─────────────────────────────────────────────────

def attend(q: np.ndarray, kv: np.ndarray, sm_scale: float,
           sink: Optional[np.ndarray] = None, d_v: int = D_LATENT):
    """One query token against its (already gathered, dequantised) rows.

    q  [H, d_qk] float32, kv [n, d_qk] float32 (n may be 0).
    Returns (out [H, d_v] float32 before the final BF16 rounding, lse [H]).

    Follows bench/bench/reference.py:516-545: logits = q.kv^T * sm_scale, a
    max-subtracted exponential, a denominator that includes exp(sink - max)
    when a sink is given, and out = attn . kv[:, :d_v].  The LSE (natural log,
    sink excluded, -inf for an empty row) follows hca/sm100/combine.cu:59-81;
    an empty row yields a zero output (combine.cu:96-100)."""
    H = q.shape[0]
    n = kv.shape[0]
    if n == 0:
        return np.zeros((H, d_v), np.float32), np.full((H,), -np.inf, np.float32)
    logits = (q.astype(np.float32) @ kv.astype(np.float32).T) * np.float32(sm_scale)
    lmax = logits.max(axis=-1, keepdims=True)
    e = np.exp(logits - lmax)
    ssum = e.sum(axis=-1, keepdims=True)
    denom = ssum.copy()
    if sink is not None:
        denom = denom + np.exp(sink.astype(np.float32).reshape(H, 1) - lmax)
    attn = e / denom
    out = attn @ kv[:, :d_v].astype(np.float32)
    lse = (lmax + np.log(ssum)).reshape(H)
    return out.astype(np.float32), lse.astype(np.float32)


def gather_rows(pool: np.ndarray, block_table_row: np.ndarray, idx: np.ndarray) -> np.ndarray:
    """Select cache entries by logical index through one request's block table.

    pool [num_pages, 64, 656] uint8; idx int (all >= 0).  Mirrors the gather
    step of the reference's sparse layer (bench/bench/reference.py:576-580),
    applied to a paged pool (paging is unpinned by the reference)."""
    idx = np.asarray(idx, dtype=np.int64)
    pages = np.asarray(block_table_row, dtype=np.int64)[idx // PAGE_ENTRIES]
    return pool[pages, idx % PAGE_ENTRIES]


def csa_sparse_decode(q, pool, block_table, indices, sm_scale, kv_len=None, sink=None):
    """CSA sparse decode.

    q [B, s_q, H, 576] float32 (BF16-representable), pool [P, 64, 656] uint8,
    block_table [B, max_pages] int32, indices [B, s_q, topk] int32 with -1 =
    padding, kv_len optional [B, s_q] int32: entries with index >= kv_len are
    not visible to that query token (the causal rule of
    bench/bench/reference.py:197-201 for speculative tokens).
    Returns (out uint16 bf16 bits [B, s_q, H, 512], lse float32 [B, s_q, H])."""
    B, s_q, H, _ = q.shape
    out = np.zeros((B, s_q, H, D_LATENT), np.uint16)
    lse = np.zeros((B, s_q, H), np.float32)
    for b in range(B):
        for j in range(s_q):
            idx = np.asarray(indices[b, j], dtype=np.int64)
            ok = idx >= 0
            if kv_len is not None:
                ok &= idx < int(kv_len[b, j])
            rows = gather_rows(pool, block_table[b], idx[ok])
            o, l = attend(q[b, j], unpack_entries(rows), sm_scale, sink)
            out[b, j] = f32_to_bf16_bits(o)
            lse[b, j] = l
    return out, lse


def hca_dense_decode(q, pool, block_table, kv_len, win, win_len, sm_scale, sink=None):
    """HCA dense decode: every compressed entry [0, kv_len) of a request plus
    its sliding window, in one softmax.

    q [B, s_q, H, 576]; pool/block_table as above; kv_len, win_len int32
    [B, s_q] (per query token, so speculative tokens can see different
    lengths); win [B, W, 656] uint8.  The concatenation order (compressed
    entries, then window) follows bench/bench/reference.py:512-514."""
    B, s_q, H, _ = q.shape
    out = np.zeros((B, s_q, H, D_LATENT), np.uint16)
    lse = np.zeros((B, s_q, H), np.float32)
    for b in range(B):
        for j in range(s_q):
            n = int(kv_len[b, j])
            w = int(win_len[b, j])
            rows = gather_rows(pool, block_table[b], np.arange(n))
            rows = np.concatenate([rows, win[b, :w]], axis=0)
            o, l = attend(q[b, j], unpack_entries(rows), sm_scale, sink)
            out[b, j] = f32_to_bf16_bits(o)
            lse[b, j] = l
    return out, lse


# ── split-KV merge ─────────────────────────────────────────────────────

def combine(partial_o, partial_lse2, sink=None):
    """LSE-weighted merge of split partials.

    partial_o [S, N, H, D] float32 (each split's output already divided by its
    own denominator), partial_lse2 [S, N, H] float32 in log2 units, -inf for an
    empty split.  Follows hca/sm100/combine.cu:59-101: lse = log2 sum 2^lse_i;
    with a sink (natural-log units) the denominator becomes
    lse + log2(1 + 2^(sink*log2e - lse)); out = sum 2^(lse_i - denom) * o_i;
    returned LSE is natural log without the sink, -inf for an empty row, whose
    output is zero.  Returns (out bf16 bits [N, H, D], lse [N, H])."""
    po = np.asarray(partial_o, np.float32)
    pl = np.asarray(partial_lse2, np.float64)
    mx = pl.max(axis=0)
    safe = np.where(np.isfinite(mx), mx, 0.0)
    ssum = np.exp2(pl - safe).sum(axis=0)
    has = ssum > 0
    with np.errstate(divide="ignore"):
        glse = np.where(has, np.log2(np.where(has, ssum, 1.0)) + safe, -np.inf)
    denom = glse.copy()
    if sink is not None:
        s2 = np.asarray(sink, np.float64).reshape(1, -1) * math.log2(math.e)
        s2 = np.broadcast_to(s2, glse.shape)
        denom = np.where(has, glse + np.log2(1.0 + np.exp2(s2 - np.where(has, glse, 0.0))), s2)
    w = np.where(np.isfinite(pl) & np.isfinite(denom)[None], np.exp2(pl - np.where(np.isfinite(denom), denom, 0.0)[None]), 0.0)
    out = (w[..., None] * po.astype(np.float64)).sum(axis=0)
    lse = np.where(has, glse * math.log(2.0), -np.inf).astype(np.float32)
    return f32_to_bf16_bits(out.astype(np.float32)), lse


# ── CSA compressor, second pass ─────────────────────────────────────────

def compress_reduce(C_a, C_b, Z_a, Z_b, B_a, B_b, m):
    """Softmax-gated reduce of the CSA compressor (cache-write side).

    C_a, C_b, Z_a, Z_b [B, n, c] float32 (BF16-representable), B_a, B_b [m, c].
    Block i combines its own m rows (a-side) with the m rows of block i-1
    (b-side): out[i] = sum_j softmax_j(Z)[j] * C[j] over the 2m positions, per
    channel; block 0 has no b-side.  Restates bench/bench/reference.py:139-155
    (the part of compressor_overlap after the projections) and the kernel
    csa/sm100/kernel.cuh:25-102.  Returns BF16 bits [B, n/m, c]."""
    B, n, c = C_a.shape
    nb = n // m
    r = lambda x: np.asarray(x, np.float32).reshape(B, nb, m, c)
    Ca, Cb, Za, Zb = r(C_a), r(C_b), r(Z_a), r(Z_b)
    Cb_s = np.concatenate([np.zeros((B, 1, m, c), np.float32), Cb[:, :-1]], axis=1)
    Zb_s = np.concatenate([np.full((B, 1, m, c), -np.inf, np.float32), Zb[:, :-1]], axis=1)
    Z = np.concatenate([Za + np.asarray(B_a, np.float32), Zb_s + np.asarray(B_b, np.float32)], axis=2)
    Cc = np.concatenate([Ca, Cb_s], axis=2)
    zmax = Z.max(axis=2, keepdims=True)
    e = np.exp(Z - zmax)
    out = (e * Cc).sum(axis=2) / e.sum(axis=2)
    return f32_to_bf16_bits(out.astype(np.float32))


@dataclass
class CompressCase:
    C_a: np.ndarray
    C_b: np.ndarray
    Z_a: np.ndarray
    Z_b: np.ndarray
    B_a: np.ndarray
    B_b: np.ndarray
    m: int


def make_compress_case(seed, B, n, c_out, m=4) -> CompressCase:
    rng = np.random.default_rng(seed)
    rn = lambda *s: bf16_round(rng.standard_normal(s, dtype=np.float32))
    return CompressCase(rn(B, n, c_out), rn(B, n, c_out), rn(B, n, c_out) * np.float32(2), rn(B, n, c_out) * np.float32(2),
                        rn(m, c_out), rn(m, c_out), m)


def hca_compress(C, Z, bias, m):
    """One-branch compressor of the HCA path (cache-write side).

    C, Z [B, n, c] float32 (BF16-representable), bias [m, c].  Block i of m rows
    becomes one row: out[i] = sum_j softmax_j(Z + bias)[j] * C[j], per channel.
    Restates the part of compressor_simple after the projections
    (bench/bench/reference.py:117-122) and the online-softmax loop of the
    reference's kernel stub (hca/sm100/kernel.cu:57-75).  Returns float32
    [B, n/m, c] (not yet rounded)."""
    B, n, c = C.shape
    nb = n // m
    Cc = np.asarray(C, np.float32).reshape(B, nb, m, c)
    Zz = np.asarray(Z, np.float32).reshape(B, nb, m, c) + np.asarray(bias, np.float32)
    zmax = Zz.max(axis=2, keepdims=True)
    e = np.exp(Zz - zmax)
    return ((e * Cc).sum(axis=2) / e.sum(axis=2)).astype(np.float32)


def quantize_insert(pool, block_table, insert_pos, rows, n_rows=None):
    """Append rows to the paged cache: rows [B, T, 576] float32 (BF16-representable)
    are quantised with this cache's recipe (`pack_entries`: FP32 absmax/448 scale per
    128 latent elements, e4m3 cast, RoPE tail kept as BF16) and written at logical
    positions insert_pos[b] .. insert_pos[b]+T-1 of request b through its block
    table.  Returns a new pool.  The quantiser follows bench/bench/decode.py:92-114;
    paging has no counterpart in the reference."""
    pool = np.array(pool, copy=True)
    B, T, _ = rows.shape
    ent = pack_entries(rows[..., :D_LATENT], rows[..., D_LATENT:])
    for b in range(B):
        t_b = T if n_rows is None else int(n_rows[b])
        for t in range(t_b):
            e = int(insert_pos[b]) + t
            pool[int(block_table[b, e // PAGE_ENTRIES]), e % PAGE_ENTRIES] = ent[b, t]
    return pool


@dataclass
class HcaCompressCase:
    C: np.ndarray
    Z: np.ndarray
    bias: np.ndarray
    m: int


def make_hca_compress_case(seed, B, n, c, m=128) -> HcaCompressCase:
    rng = np.random.default_rng(seed)
    rn = lambda *s: bf16_round(rng.standard_normal(s, dtype=np.float32))
    return HcaCompressCase(rn(B, n, c), rn(B, n, c) * np.float32(2), rn(m, c), m)


# ── the reference's own cache layout (448 e4m3 + 7 UE8M0 + 64 bf16) ─────

def quantize_ue8m0(x: np.ndarray, tile: int = 64):
    """[..., c] float32 (BF16-representable) -> (e4m3 bytes [..., c], UE8M0
    bytes [..., c/tile]).  Restates bench/bench/decode.py:92-114 line by line:
    scale = next power of two >= absmax/448, stored as its biased exponent."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    lead, c = x.shape[:-1], x.shape[-1]
    nb = c // tile
    blk = x.reshape(*lead, nb, tile)
    ratio = (np.abs(blk).max(axis=-1) / np.float32(448.0)).astype(np.float32)
    bits = ratio.view(np.int32)
    e = (bits >> 23) & 0xFF
    bump = ((bits & 0x7FFFFF) != 0).astype(np.int32)
    e_byte = np.clip(e + bump, 0, 254).astype(np.uint8)
    deq = (e_byte.astype(np.int32) << 23).view(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = blk / deq[..., None]
    scaled = np.nan_to_num(scaled, nan=0.0, posinf=448.0, neginf=-448.0)
    return f32_to_e4m3(scaled.astype(np.float32)).reshape(*lead, c), e_byte


def dequant_ue8m0(q: np.ndarray, e_byte: np.ndarray, tile: int = 64) -> np.ndarray:
    """e4m3 bytes + UE8M0 bytes -> float32; bench/bench/reference.py:422-442
    (the BF16 multiply there is exact because the scale is a power of two, as
    long as the product stays in BF16's normal range)."""
    lead, c = q.shape[:-1], q.shape[-1]
    nb = c // tile
    deq = (e_byte.astype(np.int32) << 23).view(np.float32)
    v = e4m3_to_f32(q).reshape(*lead, nb, tile) * deq.reshape(*lead, nb, 1)
    return bf16_round(v.reshape(*lead, c).astype(np.float32))


def hca_decode_ref_layout(Q, Kc, Kc_s, Kc_rope, Kswa, Kswa_s, Kswa_rope, sink, sm_scale):
    """The reference's decode step in its own cache layout, K exactly
    dequantised ("fp8_dequant" mode of bench/bench/reference.py:471-546).

    Q [B, H, c+r] float32; Kc [B, M, c] e4m3 bytes, Kc_s [B, M, c/64] UE8M0,
    Kc_rope [B, M, r] float32 (BF16-representable); Kswa* the same with W rows;
    sink [H] float32 or None.  V is the full c+r wide row
    (reference.py:543-545).  Returns (out bf16 bits [B, H, c+r], lse [B, H])."""
    B, H, dq = Q.shape
    out = np.zeros((B, H, dq), np.uint16)
    lse = np.zeros((B, H), np.float32)
    for b in range(B):
        kc = np.concatenate([dequant_ue8m0(Kc[b], Kc_s[b]), Kc_rope[b]], axis=-1)
        ks = np.concatenate([dequant_ue8m0(Kswa[b], Kswa_s[b]), Kswa_rope[b]], axis=-1)
        kv = np.concatenate([kc, ks], axis=0)
        o, l = attend(Q[b], kv, sm_scale, sink, d_v=dq)
        out[b] = f32_to_bf16_bits(o)
        lse[b] = l
    return out, lse


def rope_norm(x, positions, weight=None, eps=1e-6, n_rope=64, theta=10000.0, inverse=False):
    """Partial RoPE on the last n_rope dims, then (with `weight`) an RMS norm over the whole
    vector.  x [rows, vecs, c] float32 (BF16-representable), positions [rows].  Restates
    apply_rope (bench/bench/reference.py:35-65: split-halves pairing, freqs =
    1 / theta^(2i/n_rope), x_rot = [x1 cos - x2 sin, x1 sin + x2 cos]) followed by
    rms_norm (reference.py:68-70), the order of the reference's attention
    (reference.py:281-287); inverse=True is its output-side rotation by -position
    (reference.py:308-309).  Returns float32, not yet rounded."""
    x = np.asarray(x, np.float32)
    half = n_rope // 2
    freqs = (np.float32(1.0) / (np.float32(theta) ** (np.arange(0, n_rope, 2, dtype=np.float32) / np.float32(n_rope)))).astype(np.float32)
    pos = np.asarray(positions, np.float32) * (np.float32(-1.0) if inverse else np.float32(1.0))
    ang = (pos[:, None, None] * freqs).astype(np.float32)
    cs, sn = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    x1, x2 = x[..., -n_rope:-half], x[..., -half:]
    out = np.concatenate([x[..., :-n_rope], x1 * cs - x2 * sn, x1 * sn + x2 * cs], axis=-1).astype(np.float32)
    if weight is not None:
        rms = np.sqrt((out * out).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps)).astype(np.float32)
        out = (out / rms * np.asarray(weight, np.float32)).astype(np.float32)
    return out


# ── CSA indexer (decode form) ───────────────────────────────────────────

IDX_HEADS = 64
IDX_DIM = 128
IDX_PAGE_KEYS = 64
IDX_PAGE_BYTES = IDX_PAGE_KEYS * IDX_DIM + IDX_PAGE_KEYS * 4      # 64 x 128 e4m3 bytes, then 64 FP32 scales


def quantize_indexer_keys(K):
    """K [..., 128] float32 -> (e4m3 bytes [..., 128], FP32 scale [...]): one absmax/448
    scale per key (the recipe of bench/bench/decode.py:92-114 with one tile per key)."""
    K = np.asarray(K, np.float32)
    absmax = np.abs(K).max(axis=-1)
    scale = (absmax / np.float32(E4M3_MAX)).astype(np.float32)
    scale = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
    return f32_to_e4m3((K / scale[..., None]).astype(np.float32)), scale


def pack_indexer_pages(k8, kscale, rng=None):
    """k8 [B, n, 128] e4m3 bytes, kscale [B, n] -> (pages uint8 [P, 8448], block_table
    int32 [B, ceil(n/64)]); pages handed out in a shuffled order, unused bytes are noise."""
    rng = rng or np.random.default_rng(0)
    B, n, _ = k8.shape
    per = max(1, -(-n // IDX_PAGE_KEYS))
    P = B * per + 3
    pages = rng.integers(0, 255, size=(P, IDX_PAGE_BYTES), dtype=np.uint8)
    pages[:, IDX_PAGE_KEYS * IDX_DIM:] = 0          # noise scales must at least be finite
    bt = rng.permutation(P)[:B * per].astype(np.int32).reshape(B, per)
    for b in range(B):
        for t in range(n):
            pg, slot = bt[b, t // IDX_PAGE_KEYS], t % IDX_PAGE_KEYS
            pages[pg, slot * IDX_DIM:(slot + 1) * IDX_DIM] = k8[b, t]
            o = IDX_PAGE_KEYS * IDX_DIM + 4 * slot
            pages[pg, o:o + 4] = np.frombuffer(np.float32(kscale[b, t]).tobytes(), np.uint8)
    return pages, bt


def indexer_scores(q_fp8, q_weight, pages, block_table, n_vis):
    """score[b, t, s] = sum_h q_weight[b, t, h] * relu(q[b, t, h] . k[s]) * kscale[s] for the
    s < n_vis[b, t] visible entries, -inf beyond (Eq 16 and the causal mask of the
    reference's lightning_indexer_topk, bench/bench/reference.py:193-201; the per-key and
    per-query scales are positive and commute with the ReLU).  Returns float32
    [B, s_q, max n_vis]."""
    B, s_q = n_vis.shape
    q = e4m3_to_f32(q_fp8).astype(np.float32)                    # [B, s_q, 64, 128]
    n_max = int(n_vis.max()) if n_vis.size else 0
    out = np.full((B, s_q, n_max), -np.inf, np.float32)
    for b in range(B):
        n = int(n_vis[b].max())
        if n == 0:
            continue
        pg = block_table[b, np.arange(n) // IDX_PAGE_KEYS]
        slot = np.arange(n) % IDX_PAGE_KEYS
        raw = pages[pg]                                           # [n, 8448]
        k8 = e4m3_to_f32(raw[np.arange(n)[:, None], slot[:, None] * IDX_DIM + np.arange(IDX_DIM)[None, :]])
        ksc = np.ascontiguousarray(raw[:, IDX_PAGE_KEYS * IDX_DIM:]).view(np.float32)[np.arange(n), slot]
        for t in range(s_q):
            dots = np.einsum("hc,sc->hs", q[b, t], k8.astype(np.float32)).astype(np.float32)
            sc = (np.maximum(dots, 0) * np.asarray(q_weight[b, t], np.float32)[:, None]).sum(axis=0).astype(np.float32) * ksc
            v = int(n_vis[b, t])
            out[b, t, :v] = sc[:v]
    return out


def indexer_topk(scores, n_vis, k):
    """Indices of the k largest visible scores per (request, token), as a list of sorted
    index arrays (fewer than k when fewer are visible) - torch.topk of the masked scores
    in the reference (reference.py:203-204), as a set."""
    B, s_q = n_vis.shape
    res = [[None] * s_q for _ in range(B)]
    for b in range(B):
        for t in range(s_q):
            v = int(n_vis[b, t])
            order = np.argsort(-scores[b, t, :v], kind="stable")[:min(k, v)]
            res[b][t] = np.sort(order)
    return res


@dataclass
class IndexerCase:
    q_fp8: np.ndarray        # [B, s_q, 64, 128] e4m3 bytes
    q_scale: np.ndarray      # [B, s_q, 64] positive
    w: np.ndarray            # [B, s_q, 64] head weights
    K: np.ndarray            # [B, n, 128] float32 keys before quantisation
    n_vis: np.ndarray        # [B, s_q]


def make_indexer_case(seed, B, s_q, n, n_vis=None) -> IndexerCase:
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, s_q, IDX_HEADS, IDX_DIM), dtype=np.float32) * np.float32(2)
    q_fp8 = f32_to_e4m3(q)
    q_scale = rng.uniform(0.5, 2.0, size=(B, s_q, IDX_HEADS)).astype(np.float32)
    w = rng.standard_normal((B, s_q, IDX_HEADS)).astype(np.float32)
    K = rng.standard_normal((B, n, IDX_DIM), dtype=np.float32) * rng.uniform(0.2, 3.0, size=(B, n, 1)).astype(np.float32)
    if n_vis is None:
        n_vis = np.full((B, s_q), n, np.int32)
    return IndexerCase(q_fp8, q_scale, w, K, np.asarray(n_vis, np.int32).reshape(B, s_q))


REF_TOKEN_BYTES = 576        # 448 e4m3 latent + 64 BF16 RoPE values
REF_SCALE_BYTES = 8          # 7 UE8M0 bytes + 1 pad


def pack_ref_pages(K, K_s, K_rope, page_size, rng=None):
    """Reference-layout planes of ONE leg, K [B, M, 448] e4m3 bytes, K_s [B, M, 7]
    UE8M0, K_rope [B, M, 64] float32 (BF16-representable) -> (pages uint8
    [P, page_size*584], block_table int32 [B, ceil(M/page_size)]) in the packed page
    format of a serving engine's cache (hca/fixes.txt:79-101): per page, page_size
    tokens of [448 latent bytes | 128 RoPE bytes], then page_size x [7 scale bytes |
    1 pad byte].  Pages are handed out in a shuffled order; unused bytes are noise."""
    rng = rng or np.random.default_rng(0)
    B, M, _ = K.shape
    per = max(1, -(-M // page_size))
    P = B * per + 2
    pages = rng.integers(0, 255, size=(P, page_size * (REF_TOKEN_BYTES + REF_SCALE_BYTES)), dtype=np.uint8)
    bt = rng.permutation(P)[:B * per].astype(np.int32).reshape(B, per)
    rope_b = f32_to_bf16_bits(K_rope).view(np.uint8).reshape(B, M, 128)
    for b in range(B):
        for t in range(M):
            pg, slot = bt[b, t // page_size], t % page_size
            o = slot * REF_TOKEN_BYTES
            pages[pg, o:o + 448] = K[b, t]
            pages[pg, o + 448:o + 576] = rope_b[b, t]
            so = page_size * REF_TOKEN_BYTES + slot * REF_SCALE_BYTES
            pages[pg, so:so + 7] = K_s[b, t]
    return pages, bt


def unpack_ref_pages(pages, bt_row, n, page_size):
    """First n tokens of one request -> (K [n,448] u8, K_s [n,7] u8, K_rope [n,64] f32)."""
    K = np.zeros((n, 448), np.uint8)
    K_s = np.zeros((n, 7), np.uint8)
    rope = np.zeros((n, 64), np.float32)
    for t in range(n):
        pg, slot = bt_row[t // page_size], t % page_size
        o = slot * REF_TOKEN_BYTES
        K[t] = pages[pg, o:o + 448]
        rope[t] = bf16_bits_to_f32(np.ascontiguousarray(pages[pg, o + 448:o + 576]).view(np.uint16))
        so = page_size * REF_TOKEN_BYTES + slot * REF_SCALE_BYTES
        K_s[t] = pages[pg, so:so + 7]
    return K, K_s, rope


def hca_decode_packed_pages(Q, kv_pages, bt, m_cur, swa_pages, swa_bt, swa_len, sink, sm_scale, page_size):
    """hca_decode_ref_layout on packed pages with per-request lengths: request b
    attends to its first m_cur[b] compressed and swa_len[b] window tokens.  Only the
    addressing is new; the arithmetic is the reference decode step's."""
    B, H, dq = Q.shape
    out = np.zeros((B, H, dq), np.uint16)
    lse = np.zeros((B, H), np.float32)
    for b in range(B):
        Kc, Kc_s, Kc_r = unpack_ref_pages(kv_pages, bt[b], int(m_cur[b]), page_size)
        Ks, Ks_s, Ks_r = unpack_ref_pages(swa_pages, swa_bt[b], int(swa_len[b]), page_size)
        o, l = hca_decode_ref_layout(Q[b:b + 1], Kc[None], Kc_s[None], Kc_r[None], Ks[None], Ks_s[None], Ks_r[None], sink, sm_scale)
        out[b], lse[b] = o[0], l[0]
    return out, lse


# ── seeded synthetic inputs (shared by tests, smoke and the CPU baseline) ──

@dataclass
class CsaCase:
    q: np.ndarray            # [B, s_q, H, 576] float32, BF16-representable
    pool: np.ndarray         # [P, 64, 656] uint8
    block_table: np.ndarray  # [B, max_pages] int32
    indices: np.ndarray      # [B, s_q, topk] int32
    kv_len: np.ndarray       # [B, s_q] int32
    sm_scale: float


def make_csa_case(seed, B, s_q, H, n_entries, topk, ragged=False) -> CsaCase:
    """Draw order (numpy PCG64, fixed): q, latent, rope, page permutation, then
    per (request, token) a permutation of the visible entries.

    n_entries may be an int or a length-B sequence.  With ragged=True a query
    token whose visible context is shorter than topk gets -1 padding."""
    rng = np.random.default_rng(seed)
    n_ent = np.broadcast_to(np.asarray(n_entries, dtype=np.int64), (B,)).copy()
    pages_per = (n_ent + PAGE_ENTRIES - 1) // PAGE_ENTRIES
    max_pages = int(pages_per.max())
    P = int(pages_per.sum())
    q = bf16_round(rng.standard_normal((B, s_q, H, D_QK), dtype=np.float32))
    latent = rng.standard_normal((P, PAGE_ENTRIES, D_LATENT), dtype=np.float32)
    rope = rng.standard_normal((P, PAGE_ENTRIES, D_ROPE), dtype=np.float32)
    pool = pack_entries(latent, rope)
    perm = rng.permutation(P).astype(np.int32)
    bt = np.zeros((B, max_pages), np.int32)
    off = 0
    for b in range(B):
        bt[b, :pages_per[b]] = perm[off:off + pages_per[b]]
        off += pages_per[b]
    indices = np.full((B, s_q, topk), -1, np.int32)
    kv_len = np.zeros((B, s_q), np.int32)
    for b in range(B):
        for j in range(s_q):
            vis = int(n_ent[b]) - (s_q - 1 - j)   # later tokens see one entry more
            vis = max(vis, 0)
            kv_len[b, j] = vis
            k = min(topk, vis)
            assert ragged or k == topk, "context shorter than topk needs ragged=True"
            indices[b, j, :k] = rng.permutation(vis)[:k].astype(np.int32)
    return CsaCase(q, pool, bt, indices, kv_len, 1.0 / math.sqrt(D_QK))


@dataclass
class HcaCase:
    q: np.ndarray
    pool: np.ndarray
    block_table: np.ndarray
    kv_len: np.ndarray       # [B, s_q]
    win: np.ndarray          # [B, W, 656]
    win_len: np.ndarray      # [B, s_q]
    sink: Optional[np.ndarray]
    sm_scale: float


def make_hca_case(seed, B, s_q, H, kv_len, win_len, W=128, with_sink=False) -> HcaCase:
    """Draw order: q, latent, rope, window latent, window rope, page
    permutation, sink.  kv_len / win_len: int or length-B sequences; query
    token j of s_q sees `win_len - (s_q-1-j)` window rows."""
    rng = np.random.default_rng(seed)
    kvl = np.broadcast_to(np.asarray(kv_len, dtype=np.int64), (B,)).copy()
    wl = np.broadcast_to(np.asarray(win_len, dtype=np.int64), (B,)).copy()
    pages_per = np.maximum((kvl + PAGE_ENTRIES - 1) // PAGE_ENTRIES, 1)
    max_pages = int(pages_per.max())
    P = int(pages_per.sum())
    q = bf16_round(rng.standard_normal((B, s_q, H, D_QK), dtype=np.float32))
    pool = pack_entries(rng.standard_normal((P, PAGE_ENTRIES, D_LATENT), dtype=np.float32),
                        rng.standard_normal((P, PAGE_ENTRIES, D_ROPE), dtype=np.float32))
    win = pack_entries(rng.standard_normal((B, W, D_LATENT), dtype=np.float32),
                       rng.standard_normal((B, W, D_ROPE), dtype=np.float32))
    perm = rng.permutation(P).astype(np.int32)
    bt = np.zeros((B, max_pages), np.int32)
    off = 0
    for b in range(B):
        bt[b, :pages_per[b]] = perm[off:off + pages_per[b]]
        off += pages_per[b]
    sink = (rng.standard_normal(H).astype(np.float32) * np.float32(0.5)) if with_sink else None
    kv2 = np.repeat(kvl[:, None], s_q, axis=1).astype(np.int32)
    w2 = np.zeros((B, s_q), np.int32)
    for j in range(s_q):
        w2[:, j] = np.maximum(wl - (s_q - 1 - j), 0)
    return HcaCase(q, pool, bt, kv2, win, w2, sink, 1.0 / math.sqrt(D_QK))


@dataclass
class RefLayoutCase:
    Q: np.ndarray
    Kc: np.ndarray
    Kc_s: np.ndarray
    Kc_rope: np.ndarray
    Kswa: np.ndarray
    Kswa_s: np.ndarray
    Kswa_rope: np.ndarray
    sink: np.ndarray
    sm_scale: float


def make_ref_layout_case(seed, B, H, M_cur, swa_len, c=448, r=64) -> RefLayoutCase:
    """Inputs in the reference harness's distribution (bench/bench/decode.py:
    164-188: N(0, 0.5^2) rounded to BF16, sink N(0, 0.1^2), sm_scale =
    1/sqrt(c+r)); RoPE rotation is omitted because the kernel boundary takes
    already-rotated tensors and a rotation does not change the distribution."""
    rng = np.random.default_rng(seed)

    def rn(*shape):
        return bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.5))

    Q = rn(B, H, c + r)
    kc = rn(B, M_cur, c)
    ks = rn(B, swa_len, c)
    Kc_rope = rn(B, M_cur, r)
    Kswa_rope = rn(B, swa_len, r)
    sink = (rng.standard_normal(H).astype(np.float32) * np.float32(0.1))
    Kc, Kc_s = quantize_ue8m0(kc)
    Kswa, Kswa_s = quantize_ue8m0(ks)
    return RefLayoutCase(Q, Kc, Kc_s, Kc_rope, Kswa, Kswa_s, Kswa_rope, sink, 1.0 / math.sqrt(c + r))
