"""The CPU oracle against the reference's own outputs (golden fixtures) and
against torch's scalar-format conversions.  No GPU needed."""
import ast
import hashlib
import math
from pathlib import Path

import numpy as np
import pytest

from oracle import dsv4_oracle as orc

GOLD = Path(__file__).resolve().parent / "golden"


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def load(name):
    z = np.load(GOLD / f"{name}.npz")
    return z, ast.literal_eval(str(z["kwargs"]))


def bf16_ulp_diff(a_bits, b_bits, abs_ok=2e-6):
    """Distance in BF16 steps between two bit arrays; elements whose values
    differ by less than `abs_ok` (float32 summation-order noise on outputs that
    cancel to nearly zero) count as equal."""
    a = a_bits.astype(np.int32)
    b = b_bits.astype(np.int32)
    a = np.where(a & 0x8000, 0x8000 - a, a)
    b = np.where(b & 0x8000, 0x8000 - b, b)
    close = np.abs(orc.bf16_bits_to_f32(a_bits) - orc.bf16_bits_to_f32(b_bits)) <= abs_ok
    return np.where(close, 0, np.abs(a - b))


def test_e4m3_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 100,
        rng.standard_normal(200000).astype(np.float32),
        rng.standard_normal(50000).astype(np.float32) * 0.01,
        orc.E4M3_TABLE[:0x7F], -orc.E4M3_TABLE[:0x7F],
        ((orc.E4M3_TABLE[:0x7E].astype(np.float64) + orc.E4M3_TABLE[1:0x7F]) / 2).astype(np.float32),
        np.array([0.0, -0.0, 448.0, 449.0, 1e9, -1e9, 2 ** -10, 2 ** -9 * 0.5], np.float32),
    ])
    want = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = orc.f32_to_e4m3(x)
    # +0/-0 may differ in sign bit only for exact zeros
    assert np.array_equal(got & 0x7F, want & 0x7F)
    nz = (got & 0x7F) != 0
    assert np.array_equal(got[nz], want[nz])
    back = torch.from_numpy(got).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(orc.e4m3_to_f32(got), back)


def test_bf16_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(300000) * 10 ** rng.uniform(-6, 6, 300000)).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.f32_to_bf16_bits(x), want)


def test_pack_unpack_roundtrip():
    rng = np.random.default_rng(2)
    lat = rng.standard_normal((37, 512)).astype(np.float32)
    lat[3] = 0.0
    rope = rng.standard_normal((37, 64)).astype(np.float32)
    e = orc.pack_entries(lat, rope)
    assert e.shape == (37, orc.ENTRY_BYTES) and orc.ENTRY_BYTES == 656
    rows = orc.unpack_entries(e)
    # e4m3 keeps 3 mantissa bits: relative error <= 2^-4 of the block absmax scale
    err = np.abs(rows[:, :512] - lat).reshape(37, 4, 128).max(-1)
    assert (err <= np.abs(lat).reshape(37, 4, 128).max(-1) / 448.0 * 16 + 1e-12).all()
    assert np.array_equal(rows[:, 512:], orc.bf16_round(rope))
    # idempotence: re-quantising exactly dequantised values returns the same bytes
    e2 = orc.pack_entries(rows[:, :512], rows[:, 512:])
    assert np.array_equal(e2[:, :512], e[:, :512])


@pytest.mark.parametrize("name", ["csa_cfg0", "csa_ragged"])
def test_csa_oracle_vs_reference(name):
    z, kw = load(name)
    case = orc.make_csa_case(**kw)
    assert sha(case.q, case.pool, case.block_table, case.indices) == str(z["inputs_sha"])
    out, lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices,
                                     case.sm_scale, kv_len=case.kv_len)
    assert bf16_ulp_diff(out, z["out"]).max() <= 1
    assert (out == z["out"]).mean() > 0.98
    assert np.isfinite(lse).all()


@pytest.mark.parametrize("name", ["hca_small", "hca_nosink"])
def test_hca_oracle_vs_reference(name):
    z, kw = load(name)
    case = orc.make_hca_case(**kw)
    assert sha(case.q, case.pool, case.block_table, case.win) == str(z["inputs_sha"])
    out, lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len,
                                    case.win, case.win_len, case.sm_scale, sink=case.sink)
    assert bf16_ulp_diff(out, z["out"]).max() <= 1
    assert (out == z["out"]).mean() > 0.98


@pytest.mark.parametrize("name", ["ref_layout", "ref_layout_ragged"])
def test_ref_layout_oracle_vs_reference(name):
    z, kw = load(name)
    c = orc.make_ref_layout_case(**kw)
    assert sha(c.Q, c.Kc, c.Kc_s, c.Kc_rope, c.Kswa, c.Kswa_s, c.Kswa_rope, c.sink) == str(z["inputs_sha"])
    out, _ = orc.hca_decode_ref_layout(c.Q, c.Kc, c.Kc_s, c.Kc_rope, c.Kswa, c.Kswa_s,
                                       c.Kswa_rope, c.sink, c.sm_scale)
    assert bf16_ulp_diff(out, z["out_fp8_dequant"]).max() <= 1
    # the reference's FP8-emulating mode differs from the exact-dequant mode by
    # far more than this library's tolerance: documents why BF16 MMAs are used
    a = orc.bf16_bits_to_f32(z["out_fp8"]); b = orc.bf16_bits_to_f32(z["out_fp8_dequant"])
    assert np.abs(a - b).max() < 5e-2


def test_lse_and_combine_consistency():
    """Splitting the rows of one softmax and merging with `combine` gives the
    unsplit result (the algebra of hca/sm100/combine.cu:59-101)."""
    rng = np.random.default_rng(5)
    H, n = 8, 300
    q = orc.bf16_round(rng.standard_normal((H, 576)).astype(np.float32))
    kv = rng.standard_normal((n, 576)).astype(np.float32)
    sink = rng.standard_normal(H).astype(np.float32)
    sc = 1 / math.sqrt(576)
    for snk in (None, sink):
        full, lse = orc.attend(q, kv, sc, snk)
        cuts = [0, 64, 64, 200, 300]            # includes an empty split
        po, pl = [], []
        for a, b in zip(cuts[:-1], cuts[1:]):
            o, l = orc.attend(q, kv[a:b], sc, None)
            po.append(o)
            pl.append(l * math.log2(math.e))
        out, lse2 = orc.combine(np.stack(po)[:, None], np.stack(pl)[:, None], snk)
        assert np.allclose(lse2[0], lse, rtol=1e-5, atol=1e-5)
        assert bf16_ulp_diff(out[0], orc.f32_to_bf16_bits(full)).max() <= 1
    # all-empty
    out, lse2 = orc.combine(np.zeros((2, 1, H, 512), np.float32), np.full((2, 1, H), -np.inf, np.float32), sink)
    assert (out == 0).all() and np.isneginf(lse2).all()


def test_empty_and_padding_rows():
    case = orc.make_csa_case(seed=7, B=2, s_q=1, H=4, n_entries=[5, 130], topk=64, ragged=True)
    case.indices[0, 0, :] = -1                   # a request with nothing visible
    out, lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale)
    assert (out[0] == 0).all() and np.isneginf(lse[0]).all()
    assert np.isfinite(lse[1]).all()
    # padding position does not matter
    idx2 = case.indices.copy()
    idx2[1, 0] = np.roll(idx2[1, 0], 7)
    out2, lse2 = orc.csa_sparse_decode(case.q, case.pool, case.block_table, idx2, case.sm_scale)
    assert bf16_ulp_diff(out2[1], out[1]).max() <= 1


@pytest.mark.parametrize("name", ["csa_compress", "csa_compress_odd"])
def test_compress_reduce_oracle_vs_reference(name):
    z, kw = load(name)
    c = orc.make_compress_case(**kw)
    assert sha(c.C_a, c.C_b, c.Z_a, c.Z_b, c.B_a, c.B_b) == str(z["inputs_sha"])
    out = orc.compress_reduce(c.C_a, c.C_b, c.Z_a, c.Z_b, c.B_a, c.B_b, c.m)
    assert out.shape == z["out"].shape
    assert bf16_ulp_diff(out, z["out"]).max() <= 1


@pytest.mark.parametrize("name", ["hca_compress", "hca_compress_m16"])
def test_hca_compress_oracle_vs_reference(name):
    z, kw = load(name)
    c = orc.make_hca_compress_case(**kw)
    assert sha(c.C, c.Z, c.bias) == str(z["inputs_sha"])
    out = orc.hca_compress(c.C, c.Z, c.bias, c.m)
    assert out.shape == z["out"].shape
    np.testing.assert_allclose(out, z["out"], rtol=2e-5, atol=2e-6)


def test_quantize_insert_places_entries():
    """Rows appended through the block table read back (unpack_entries) as the
    quantiser's round trip of the rows; untouched entries keep their bytes."""
    rng = np.random.default_rng(11)
    B, T = 3, 70
    pages_per = 3
    bt = rng.permutation(B * pages_per).astype(np.int32).reshape(B, pages_per)
    pool = rng.integers(0, 255, size=(B * pages_per, orc.PAGE_ENTRIES, orc.ENTRY_BYTES), dtype=np.uint8)
    rows = orc.bf16_round(rng.standard_normal((B, T, orc.D_QK), dtype=np.float32))
    rows[0, 0, :128] = 0           # a block of zeros gets scale 1
    pos = np.array([0, 60, 100], np.int32)
    n_rows = np.array([70, 64, 5], np.int32)
    new = orc.quantize_insert(pool, bt, pos, rows, n_rows)
    want = orc.unpack_entries(orc.pack_entries(rows[..., :512], rows[..., 512:]))
    changed = np.zeros(pool.shape[:2], bool)
    for b in range(B):
        for t in range(n_rows[b]):
            e = pos[b] + t
            got = orc.unpack_entries(new[bt[b, e // 64], e % 64])
            np.testing.assert_array_equal(got, want[b, t])
            changed[bt[b, e // 64], e % 64] = True
    assert np.array_equal(new[~changed], pool[~changed])
    assert np.abs(want[..., :512] - rows[..., :512]).max() <= np.abs(rows).max() / 16 + 1e-6   # e4m3: 3 mantissa bits
    assert np.array_equal(want[..., 512:], rows[..., 512:])


def test_packed_pages_oracle_matches_reference_output():
    """The reference-layout golden case repacked into cache pages (page sizes 16 and 64)
    decodes to the reference's own output: packing is addressing only."""
    z, kw = load("ref_layout_ragged")
    c = orc.make_ref_layout_case(**kw)
    B = c.Q.shape[0]
    for ps in (16, 64):
        rng = np.random.default_rng(5)
        kv_pages, bt = orc.pack_ref_pages(c.Kc, c.Kc_s, c.Kc_rope, ps, rng)
        sw_pages, sbt = orc.pack_ref_pages(c.Kswa, c.Kswa_s, c.Kswa_rope, ps, rng)
        m_cur = np.full(B, c.Kc.shape[1], np.int32)
        swa = np.full(B, c.Kswa.shape[1], np.int32)
        out, _ = orc.hca_decode_packed_pages(c.Q, kv_pages, bt, m_cur, sw_pages, sbt, swa, c.sink, c.sm_scale, ps)
        assert bf16_ulp_diff(out, z["out_fp8_dequant"]).max() <= 1
        # shorter per-request lengths = the same attention over a prefix
        m2 = np.array([40, 3], np.int32)[:B]
        s2 = np.array([0, 19], np.int32)[:B]
        out2, lse2 = orc.hca_decode_packed_pages(c.Q, kv_pages, bt, m2, sw_pages, sbt, s2, c.sink, c.sm_scale, ps)
        for b in range(B):
            want, wl = orc.hca_decode_ref_layout(c.Q[b:b + 1], c.Kc[b:b + 1, :m2[b]], c.Kc_s[b:b + 1, :m2[b]], c.Kc_rope[b:b + 1, :m2[b]],
                                                 c.Kswa[b:b + 1, :s2[b]], c.Kswa_s[b:b + 1, :s2[b]], c.Kswa_rope[b:b + 1, :s2[b]],
                                                 c.sink, c.sm_scale)
            assert np.array_equal(out2[b], want[0]) and np.array_equal(lse2[b], wl[0])


@pytest.mark.parametrize("name", ["rope_norm_q576", "rope_norm_o512"])
def test_rope_norm_oracle_vs_reference(name):
    from tests.golden.gen_golden import make_rope_norm_inputs
    z, kw = load(name)
    x, pos, w = make_rope_norm_inputs(**kw)
    assert sha(x, pos, w) == str(z["inputs_sha"])
    # angles reach 1e5 rad in the second case: float32 pow/cos differ between libraries in the last place
    tol = dict(rtol=1e-4, atol=5e-3 if kw["max_pos"] > 10000 else 5e-4)
    np.testing.assert_allclose(orc.rope_norm(x, pos, w, eps=1e-6), z["q"], **tol)
    np.testing.assert_allclose(orc.rope_norm(x, pos, None, inverse=True), z["o"], **tol)
    # rotating forth and back is the identity
    back = orc.rope_norm(orc.rope_norm(x, pos), pos, inverse=True)
    np.testing.assert_allclose(back, x, rtol=1e-4, atol=1e-4)


def indexer_inputs(c, rng):
    """Device-facing inputs of an IndexerCase: quantised keys in pages, folded weights."""
    k8, ksc = orc.quantize_indexer_keys(c.K)
    pages, bt = orc.pack_indexer_pages(k8, ksc, rng)
    return pages, bt, (c.w * c.q_scale).astype(np.float32)


def test_indexer_oracle_vs_reference():
    z, kw = load("indexer_topk")
    kwc = {k: v for k, v in kw.items() if k not in ("m", "top_k", "tokens")}
    c = orc.make_indexer_case(**kwc)
    assert sha(c.q_fp8, c.q_scale, c.w, c.K) == str(z["inputs_sha"])
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(1))
    n_vis = z["n_vis"]
    scores = orc.indexer_scores(c.q_fp8, qw, pages, bt, n_vis)
    sel = orc.indexer_topk(scores, n_vis, kw["top_k"])
    for b in range(n_vis.shape[0]):
        for t in range(n_vis.shape[1]):
            assert np.array_equal(sel[b][t], np.sort(z["sel"][b, t])), (b, t)
            assert (z["sel"][b, t] < n_vis[b, t]).all()
            # the reference lists its selection best first
            ref_scores = scores[b, t, z["sel"][b, t]]
            assert (np.diff(ref_scores) <= 1e-4 * np.abs(ref_scores[:-1]) + 1e-6).all()
