"""GPU parity of the cache-write side: the HCA compressor and the
quantise-and-insert step, through the C ABI, against the CPU oracle and the
committed reference outputs.  Run with `-m gpu` on a B200."""
import ast
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import dsv4_oracle as orc  # noqa: E402
from tests import gpu_util as gu  # noqa: E402

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as d
    return d


def golden(name):
    z = np.load(GOLD / f"{name}.npz")
    return z, ast.literal_eval(str(z["kwargs"]))


def bf(a):
    return gu.dev(a, torch.bfloat16)


def make_pool(rng, B, pages_per):
    bt = rng.permutation(B * pages_per).astype(np.int32).reshape(B, pages_per)
    pool = rng.integers(0, 255, size=(B * pages_per, orc.PAGE_ENTRIES, orc.ENTRY_BYTES), dtype=np.uint8)
    return pool, bt


@pytest.mark.parametrize("name", ["hca_compress", "hca_compress_m16"])
def test_hca_compress_vs_reference_outputs(lib, name):
    """Dense BF16 output against the reference's compressor_simple (float32) rounded to
    BF16: at most 1 BF16 ulp apart."""
    z, kw = golden(name)
    c = orc.make_hca_compress_case(**kw)
    out = lib.hca_compress_fwd(bf(c.C), bf(c.Z), bf(c.bias), c.m)
    torch.cuda.synchronize()
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    from tests.test_oracle import bf16_ulp_diff
    assert got.shape == z["out"].shape
    assert bf16_ulp_diff(got, orc.f32_to_bf16_bits(z["out"])).max() <= 1
    assert bf16_ulp_diff(got, orc.f32_to_bf16_bits(orc.hca_compress(c.C, c.Z, c.bias, c.m))).max() <= 1


def test_kv_quantize_insert_bit_exact(lib):
    """Entries written by the GPU quantiser are byte-identical to the CPU restatement's,
    ragged row counts and page-crossing positions included; other entries are untouched."""
    rng = np.random.default_rng(21)
    B, T = 4, 150
    pool, bt = make_pool(rng, B, 4)
    rows = orc.bf16_round(rng.standard_normal((B, T, orc.D_QK), dtype=np.float32) * rng.uniform(0.01, 30, size=(B, T, 1)).astype(np.float32))
    rows[1, 3, 128:256] = 0
    rows[2, 7] = 0
    pos = np.array([0, 63, 100, 17], np.int32)
    n_rows = np.array([150, 129, 0, 64], np.int32)
    want = orc.quantize_insert(pool, bt, pos, rows, n_rows)
    d_pool = gu.dev(pool)
    status = lib.new_status(d_pool.device)
    lib.kv_quantize_insert(bf(rows), d_pool, gu.dev(bt), gu.dev(pos), n_rows=gu.dev(n_rows), status=status)
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    assert np.array_equal(d_pool.cpu().numpy(), want)
    # without n_rows: all T rows
    pos2 = np.array([10, 0, 50, 100], np.int32)
    want2 = orc.quantize_insert(pool, bt, pos2, rows)
    d_pool2 = gu.dev(pool)
    lib.kv_quantize_insert(bf(rows), d_pool2, gu.dev(bt), gu.dev(pos2))
    torch.cuda.synchronize()
    assert np.array_equal(d_pool2.cpu().numpy(), want2)


def test_kv_quantize_insert_out_of_range_is_reported_not_written(lib):
    rng = np.random.default_rng(22)
    B, T = 2, 8
    pool, bt = make_pool(rng, B, 2)                     # 128 entries per request
    rows = orc.bf16_round(rng.standard_normal((B, T, orc.D_QK), dtype=np.float32))
    pos = np.array([0, 124], np.int32)                  # request 1: rows 4..7 fall off the block table
    d_pool = gu.dev(pool)
    status = lib.new_status(d_pool.device)
    lib.kv_quantize_insert(bf(rows), d_pool, gu.dev(bt), gu.dev(pos), status=status)
    torch.cuda.synchronize()
    st = status.cpu().tolist()
    assert st[0] == 16 and st[1] == 1 and 128 <= st[2] < 132
    want = orc.quantize_insert(pool, bt, pos, rows, np.array([8, 4], np.int32))
    assert np.array_equal(d_pool.cpu().numpy(), want)
    with pytest.raises(ValueError):
        lib.kv_quantize_insert(bf(rows)[..., :512].contiguous(), d_pool, gu.dev(bt), gu.dev(pos))


def test_hca_compress_fused_insert_equals_two_steps(lib):
    """The fused compressor + quantiser + insert writes the same bytes as the dense
    compressor output followed by kv_quantize_insert, and those entries decode (through the
    oracle's dequantiser) to the oracle's compressor output within e4m3 resolution."""
    rng = np.random.default_rng(23)
    B, n, m = 3, 128 * 5, 128
    c = orc.make_hca_compress_case(seed=24, B=B, n=n, c=orc.D_QK, m=m)
    pool, bt = make_pool(rng, B, 3)
    pos = np.array([0, 62, 120], np.int32)
    d_bt, d_pos = gu.dev(bt), gu.dev(pos)
    fused = gu.dev(pool)
    status = lib.new_status(fused.device)
    out = lib.hca_compress_fwd(bf(c.C), bf(c.Z), bf(c.bias), m, kv_pool=fused, block_table=d_bt, insert_pos=d_pos, status=status)
    two = gu.dev(pool)
    lib.kv_quantize_insert(out, two, d_bt, d_pos)
    only = gu.dev(pool)
    assert lib.hca_compress_fwd(bf(c.C), bf(c.Z), bf(c.bias), m, kv_pool=only, block_table=d_bt, insert_pos=d_pos, want_out=False) is None
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    assert torch.equal(fused, two) and torch.equal(fused, only)
    want = orc.hca_compress(c.C, c.Z, c.bias, m)                       # float32 [B, 5, 576]
    new = fused.cpu().numpy()
    for b in range(B):
        for i in range(n // m):
            e = pos[b] + i
            got = orc.unpack_entries(new[bt[b, e // 64], e % 64])
            blk_max = np.abs(want[b, i, :512]).reshape(4, 128).max(axis=1).repeat(128)
            assert (np.abs(got[:512] - want[b, i, :512]) <= blk_max / 16 + 1e-6).all()
            assert np.abs(got[512:] - want[b, i, 512:]).max() <= 2e-2
    # and the entries the oracle's own quantiser makes from the GPU's dense output are the same bytes
    want_pool = orc.quantize_insert(pool, bt, pos, out.float().cpu().numpy())
    assert np.array_equal(new, want_pool)


def test_hca_compress_invalid_arguments(lib):
    c = orc.make_hca_compress_case(seed=25, B=1, n=32, c=40, m=16)
    with pytest.raises(ValueError):
        lib.hca_compress_fwd(bf(c.C), bf(c.Z), bf(c.bias)[:8].contiguous(), 16)          # bias rows != m
    with pytest.raises(ValueError):
        lib.hca_compress_fwd(bf(c.C)[:, :30].contiguous(), bf(c.Z)[:, :30].contiguous(), bf(c.bias), 16)   # n % m
    with pytest.raises(ValueError):
        lib.hca_compress_fwd(bf(c.C).float(), bf(c.Z), bf(c.bias), 16)
    pool, bt = make_pool(np.random.default_rng(1), 1, 1)
    with pytest.raises(ValueError):                                                       # insert needs c == 576
        lib.hca_compress_fwd(bf(c.C), bf(c.Z), bf(c.bias), 16, kv_pool=gu.dev(pool), block_table=gu.dev(bt),
                             insert_pos=gu.dev(np.zeros(1, np.int32)))


def test_written_entries_are_read_by_the_decode_kernel(lib):
    """Write side and read side agree on the layout: a cache filled by kv_quantize_insert is
    attended to by the HCA decode kernel with the same result as the oracle on the rows."""
    rng = np.random.default_rng(26)
    B, H, n_ent = 2, 16, 100
    rows = orc.bf16_round(rng.standard_normal((B, n_ent, orc.D_QK), dtype=np.float32))
    pool, bt = make_pool(rng, B, 2)
    d_pool = gu.dev(pool)
    lib.kv_quantize_insert(bf(rows), d_pool, gu.dev(bt), gu.dev(np.zeros(B, np.int32)))
    q = orc.bf16_round(rng.standard_normal((B, 1, H, orc.D_QK), dtype=np.float32))
    kv_len = np.full((B, 1), n_ent, np.int32)
    win = np.zeros((B, 128, orc.ENTRY_BYTES), np.uint8)
    win_len = np.zeros((B, 1), np.int32)
    sm = orc.D_QK ** -0.5
    out, lse = lib.hca_dense_decode(bf(q), d_pool, gu.dev(bt), gu.dev(kv_len), gu.dev(win), gu.dev(win_len), sm)
    torch.cuda.synchronize()
    want_pool = orc.quantize_insert(pool, bt, np.zeros(B, np.int32), rows)
    want_out, want_lse = orc.hca_dense_decode(q, want_pool, bt, kv_len, win, win_len, sm)
    gu.check_out(gu.out_to_f32(out), want_out, "decode over inserted entries")
    gu.check_lse(lse.cpu().numpy(), want_lse, "decode over inserted entries")


@pytest.mark.parametrize("name", ["rope_norm_q576", "rope_norm_o512"])
def test_rope_norm_vs_reference_outputs(lib, name):
    """Query pre-pass (RoPE then RMS norm) and output post-pass (inverse RoPE) against the
    reference's apply_rope / rms_norm outputs: within 2 BF16 ulps (a few at large angles,
    where float32 cos/sin of different libraries differ in the last place)."""
    from tests.golden.gen_golden import make_rope_norm_inputs
    from tests.test_oracle import bf16_ulp_diff
    z, kw = golden(name)
    x, pos, w = make_rope_norm_inputs(**kw)
    dx, dpos, dw = bf(x), gu.dev(pos), bf(w)
    q = lib.rope_norm(dx, dpos, norm_weight=dw, eps=1e-6)
    o = lib.rope_norm(dx, dpos, inverse=True)
    torch.cuda.synchronize()
    bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    big = kw["max_pos"] > 10000
    for got, want in ((q, z["q"]), (o, z["o"])):
        d = bf16_ulp_diff(bits(got), orc.f32_to_bf16_bits(want), abs_ok=5e-3 if big else 2e-6)
        assert d.max() <= 2 and (d > 1).mean() < 1e-3
    # in place, and forth-and-back = identity up to BF16 rounding of the rotated pair
    y = dx.clone()
    lib.rope_norm(y, dpos, out=y)
    lib.rope_norm(y, dpos, inverse=True, out=y)
    torch.cuda.synchronize()
    assert torch.equal(y[..., :-64], dx[..., :-64])
    assert (y[..., -64:].float() - dx[..., -64:].float()).abs().max().item() <= 4e-2
    with pytest.raises(ValueError):
        lib.rope_norm(dx[..., :100].contiguous(), dpos)
