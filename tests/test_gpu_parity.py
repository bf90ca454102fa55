"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU
oracle and the committed reference outputs.  Run with `-m gpu` on a B200."""
import ast
import math
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


def run_csa(lib, case, **kw):
    st = lib.new_status("cuda")
    args = gu.csa_to_dev(case)
    out, lse = lib.csa_sparse_decode(status=st, **args, **kw)
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0], f"kernel reported a bounded-wait timeout: {st.cpu().tolist()}"
    return gu.out_to_f32(out), lse.cpu().numpy()


def run_hca(lib, case, **kw):
    st = lib.new_status("cuda")
    args = gu.hca_to_dev(case)
    out, lse = lib.hca_dense_decode(status=st, **args, **kw)
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0], f"kernel reported a bounded-wait timeout: {st.cpu().tolist()}"
    return gu.out_to_f32(out), lse.cpu().numpy()


@pytest.mark.parametrize("impl", ["simt", "mma"])
@pytest.mark.parametrize("name", ["csa_cfg0", "csa_ragged"])
def test_csa_vs_reference_outputs(lib, name, impl):
    z, kw = golden(name)
    case = orc.make_csa_case(**kw)
    out, lse = run_csa(lib, case, impl=impl, num_splits=1)
    gu.check_out(out, z["out"], f"{name}/{impl} vs reference")
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices,
                                               case.sm_scale, kv_len=case.kv_len)
    gu.check_out(out, want_out, f"{name}/{impl} vs oracle")
    gu.check_lse(lse, want_lse, f"{name}/{impl}")


@pytest.mark.parametrize("impl", ["simt", "mma"])
@pytest.mark.parametrize("name", ["hca_small", "hca_nosink"])
def test_hca_vs_reference_outputs(lib, name, impl):
    z, kw = golden(name)
    case = orc.make_hca_case(**kw)
    out, lse = run_hca(lib, case, impl=impl, num_splits=1)
    gu.check_out(out, z["out"], f"{name}/{impl} vs reference")
    want_out, want_lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len, case.win,
                                              case.win_len, case.sm_scale, sink=case.sink)
    gu.check_out(out, want_out, f"{name}/{impl} vs oracle")
    gu.check_lse(lse, want_lse, f"{name}/{impl}")


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_csa_split_kv(lib, splits):
    case = orc.make_csa_case(seed=11, B=3, s_q=2, H=32, n_entries=[700, 1500, 90], topk=512, ragged=True)
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices,
                                               case.sm_scale, kv_len=case.kv_len)
    out, lse = run_csa(lib, case, num_splits=splits)
    gu.check_out(out, want_out, f"csa splits={splits}")
    gu.check_lse(lse, want_lse, f"csa splits={splits}")


@pytest.mark.parametrize("splits", [2, 5])
def test_hca_split_kv_with_sink(lib, splits):
    case = orc.make_hca_case(seed=12, B=2, s_q=2, H=128, kv_len=[782, 333], win_len=[128, 40], with_sink=True)
    want_out, want_lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len, case.win,
                                              case.win_len, case.sm_scale, sink=case.sink)
    out, lse = run_hca(lib, case, num_splits=splits)
    gu.check_out(out, want_out, f"hca splits={splits}")
    gu.check_lse(lse, want_lse, f"hca splits={splits}")


def test_csa_h128_paged_like_config1(lib):
    """Config-1 shape at a reduced batch: H=128, 768 entries in 64-entry pages
    behind a random block table, top-k 512, no split."""
    case = orc.make_csa_case(seed=13, B=4, s_q=1, H=128, n_entries=768, topk=512)
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale)
    out, lse = run_csa(lib, case, num_splits=1)
    e = gu.check_out(out, want_out, "csa H=128")
    gu.check_lse(lse, want_lse, "csa H=128")
    print("csa H=128 max/mean abs err", e)


def test_hca_h128_like_config2(lib):
    case = orc.make_hca_case(seed=14, B=3, s_q=1, H=128, kv_len=782, win_len=128)
    want_out, want_lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len, case.win,
                                              case.win_len, case.sm_scale)
    out, lse = run_hca(lib, case, num_splits=1)
    e = gu.check_out(out, want_out, "hca H=128")
    gu.check_lse(lse, want_lse, "hca H=128")
    print("hca H=128 max/mean abs err", e)


def test_padding_anywhere_and_empty_rows(lib):
    case = orc.make_csa_case(seed=15, B=3, s_q=1, H=16, n_entries=[5, 130, 400], topk=192, ragged=True)
    case.indices[0, 0, :] = -1                       # nothing visible at all
    rng = np.random.default_rng(0)
    case.indices[2, 0] = rng.permutation(case.indices[2, 0])     # padding scattered, not at the tail
    case.indices[2, 0, ::3] = -1
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices,
                                               case.sm_scale, kv_len=case.kv_len)
    for splits in (1, 2):
        out, lse = run_csa(lib, case, num_splits=splits)
        gu.check_out(out, want_out, f"padding splits={splits}")
        gu.check_lse(lse, want_lse, f"padding splits={splits}")
        assert (out[0] == 0).all() and np.isneginf(lse[0]).all()


def test_growing_maximum_rescales_accumulator(lib):
    """Later tiles carry much larger logits than earlier ones, so the running
    reference maximum must move and the accumulator in tensor memory must be
    rescaled several times."""
    B, H, n = 1, 128, 512
    rng = np.random.default_rng(21)
    q = orc.bf16_round(rng.standard_normal((B, 1, H, 576)).astype(np.float32))
    lat = rng.standard_normal((n, 512)).astype(np.float32)
    rope = rng.standard_normal((n, 64)).astype(np.float32)
    grow = (1.0 + 0.5 * (np.arange(n) // 64)).astype(np.float32)[:, None]   # x1 ... x4.5 per tile
    lat *= grow
    rope *= grow
    pool = orc.pack_entries(lat.reshape(n // 64, 64, 512), rope.reshape(n // 64, 64, 64))
    bt = np.arange(n // 64, dtype=np.int32)[None]
    idx = np.arange(n, dtype=np.int32)[None, None]
    sc = 1 / math.sqrt(576)
    want_out, want_lse = orc.csa_sparse_decode(q, pool, bt, idx, sc)
    case = orc.CsaCase(q, pool, bt, idx, np.full((1, 1), n, np.int32), sc)
    for impl in ("simt", "mma"):
        out, lse = run_csa(lib, case, impl=impl, num_splits=1)
        # outputs are O(40) here: compare relative to the value scale
        scale = np.abs(gu.bits_to_f32(want_out)).max()
        err = np.abs(out - gu.bits_to_f32(want_out)) / scale
        assert err.max() < 2e-2, (impl, err.max())
        # the LSE is ~16 here and BF16 rounding of K moves it by ~0.02
        assert np.abs(lse - want_lse).max() <= 3e-3 * np.abs(want_lse).max(), impl


def test_combine_kernel_vs_oracle(lib):
    rng = np.random.default_rng(31)
    S, N, H = 5, 3, 20
    po = rng.standard_normal((S, N, H, 512)).astype(np.float32)
    pl = (rng.standard_normal((S, N, H)) * 3).astype(np.float32)
    pl[1] = -np.inf                      # an empty split
    pl[:, 2, 7] = -np.inf                # a fully empty (row, head)
    po[1] = np.nan                       # empty splits may hold anything
    sink = rng.standard_normal(H).astype(np.float32)
    for snk in (None, sink):
        want_out, want_lse = orc.combine(np.nan_to_num(po), pl, snk)
        out, lse = lib.combine(gu.dev(po), gu.dev(pl), attn_sink=None if snk is None else gu.dev(snk))
        torch.cuda.synchronize()
        got = gu.out_to_f32(out)
        assert np.abs(got - gu.bits_to_f32(want_out)).max() <= 2e-2 * max(1.0, np.abs(gu.bits_to_f32(want_out)).max())
        gu.check_lse(lse.cpu().numpy(), want_lse, "combine")
        assert (got[2, 7] == 0).all()


@pytest.mark.parametrize("name", ["ref_layout", "ref_layout_ragged"])
def test_reference_entry_point_on_reference_layout(lib, name):
    """hca_decode_fwd, the reference's own symbol and cache layout, against the
    reference's fp8_dequant output with the reference harness's tolerance
    (bench/bench/decode.py:48-53,328-330) and this library's tighter one."""
    z, kw = golden(name)
    c = orc.make_ref_layout_case(**kw)
    d = gu.dev
    O = lib.hca_decode_fwd(d(c.Q, torch.bfloat16), d(c.Kc), d(c.Kc_s), d(c.Kc_rope, torch.bfloat16),
                           d(c.Kswa), d(c.Kswa_s), d(c.Kswa_rope, torch.bfloat16), d(c.sink), c.sm_scale,
                           M_cur=kw["M_cur"], swa_len=kw["swa_len"])
    torch.cuda.synchronize()
    got = gu.out_to_f32(O)
    want = gu.bits_to_f32(z["out_fp8_dequant"])
    err = np.abs(got - want)
    assert err.max() <= 1.5e-2 or (err / np.maximum(np.abs(want), 1e-8)).max() <= 5e-2
    gu.check_out(got, z["out_fp8_dequant"], name)


def test_invalid_arguments_are_rejected(lib):
    case = orc.make_csa_case(seed=1, B=1, s_q=1, H=4, n_entries=64, topk=64)
    args = gu.csa_to_dev(case)
    with pytest.raises(lib.Dsv4Error):
        lib.csa_sparse_decode(**{**args, "sm_scale": float("nan")})
    with pytest.raises(ValueError):
        lib.csa_sparse_decode(**{**args, "q": args["q"].float()})
    with pytest.raises(ValueError):
        lib.csa_sparse_decode(**args, num_splits=65)
    import ctypes as C
    assert lib.LIB.dsv4_csa_sparse_decode_fwd(None, None) == 1
    assert lib.LIB.hca_decode_fwd(*([None] * 11), C.c_float(1.0), 1, 128, 512, 64, 128, 0, None) == 1
    torch.cuda.synchronize()


def test_combine_kernel_vs_reference_kernel(lib):
    """This library's merge against the reference project's own merge kernel
    (hca/sm100/combine.cu, compiled from the reference sources into
    oracle/_ref by oracle/build_ref.py) on the same partials: bit-exact LSE
    pattern and BF16 outputs within one rounding step."""
    import ctypes as C
    so = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libref_combine.so"
    if not so.exists():
        pytest.skip("oracle/_ref not built (needs the reference sources)")
    ref = C.CDLL(str(so))
    ref.ref_hca_combine.restype = C.c_int
    ref.ref_hca_combine.argtypes = [C.c_int] * 3 + [C.c_void_p] * 6
    rng = np.random.default_rng(41)
    for S, B, H in ((8, 4, 128), (33, 2, 24), (1, 3, 8)):
        po = gu.dev(rng.standard_normal((S, B, H, 512)).astype(np.float32))
        pl_np = (rng.standard_normal((S, B, H)) * 4).astype(np.float32)
        if S > 2:
            pl_np[2] = -np.inf
        pl = gu.dev(pl_np)
        sink = gu.dev(rng.standard_normal(H).astype(np.float32))
        for snk in (None, sink):
            out_ref = torch.empty(B, H, 512, dtype=torch.bfloat16, device="cuda")
            lse_ref = torch.empty(B, H, dtype=torch.float32, device="cuda")
            rc = ref.ref_hca_combine(B, H, S, po.data_ptr(), pl.data_ptr(), out_ref.data_ptr(), lse_ref.data_ptr(),
                                     None if snk is None else snk.data_ptr(), None)
            assert rc == 0
            out, lse = lib.combine(po, pl, attn_sink=snk)
            torch.cuda.synchronize()
            a, b = out.float(), out_ref.float()
            assert torch.allclose(a, b, rtol=2 ** -7, atol=1e-6), (S, B, H, (a - b).abs().max().item())
            assert torch.allclose(lse, lse_ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", ["csa_compress", "csa_compress_odd"])
def test_compress_reduce_vs_reference_outputs(lib, name):
    z, kw = golden(name)
    c = orc.make_compress_case(**kw)
    bf = lambda a: gu.dev(a, torch.bfloat16)
    out = lib.csa_compress_reduce_fwd(bf(c.C_a), bf(c.C_b), bf(c.Z_a), bf(c.Z_b), bf(c.B_a), bf(c.B_b), c.m)
    torch.cuda.synchronize()
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    from tests.test_oracle import bf16_ulp_diff
    assert bf16_ulp_diff(got, z["out"]).max() <= 1
    assert bf16_ulp_diff(got, orc.compress_reduce(c.C_a, c.C_b, c.Z_a, c.Z_b, c.B_a, c.B_b, c.m)).max() <= 1


def test_compress_reduce_vs_reference_kernel_and_errors(lib):
    """Against the reference project's own kernel (csa/sm100/kernel.cuh, built
    from the reference sources into oracle/_ref) at a realistic size, plus the
    argument checks of the reference's operator (csa/interface.h:30-52,79-83)."""
    import ctypes as C
    c = orc.make_compress_case(seed=61, B=2, n=4096, c_out=512)
    bf = lambda a: gu.dev(a, torch.bfloat16)
    t = [bf(x) for x in (c.C_a, c.C_b, c.Z_a, c.Z_b, c.B_a, c.B_b)]
    out = lib.csa_compress_reduce_fwd(*t, 4)
    want = orc.compress_reduce(c.C_a, c.C_b, c.Z_a, c.Z_b, c.B_a, c.B_b, 4)
    from tests.test_oracle import bf16_ulp_diff
    assert bf16_ulp_diff(out.view(torch.int16).cpu().numpy().view(np.uint16), want).max() <= 1
    so = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libref_csa.so"
    if so.exists():
        ref = C.CDLL(str(so))
        ref.ref_csa_compress_reduce.restype = C.c_int
        ref.ref_csa_compress_reduce.argtypes = [C.c_int] * 4 + [C.c_void_p] * 8
        out_ref = torch.empty_like(out)
        assert ref.ref_csa_compress_reduce(2, 4096, 512, 4, *[x.data_ptr() for x in t], out_ref.data_ptr(), None) == 0
        torch.cuda.synchronize()
        a = out.view(torch.int16).cpu().numpy().view(np.uint16)
        b = out_ref.view(torch.int16).cpu().numpy().view(np.uint16)
        assert bf16_ulp_diff(a, b).max() <= 1 and (a == b).mean() > 0.99
    with pytest.raises(ValueError, match="unsupported m"):
        lib.csa_compress_reduce_fwd(*[x if x.dim() == 3 else x[:2].contiguous() for x in t], 2)
    with pytest.raises(ValueError, match="bf16"):
        lib.csa_compress_reduce_fwd(t[0].float(), *t[1:], 4)
    with pytest.raises(ValueError, match="divisible"):
        lib.csa_compress_reduce_fwd(*[x[:, :4095].contiguous() if x.dim() == 3 else x for x in t], 4)


def test_more_than_128_heads_and_partial_head_group(lib):
    """H = 192: two groups of 128 head rows, the second only half used."""
    case = orc.make_csa_case(seed=71, B=2, s_q=1, H=192, n_entries=300, topk=256)
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale)
    for splits in (1, 2):
        out, lse = run_csa(lib, case, num_splits=splits)
        gu.check_out(out, want_out, f"H=192 splits={splits}")
        gu.check_lse(lse, want_lse, f"H=192 splits={splits}")


def test_topk_len_and_more_splits_than_tiles(lib):
    """Ragged index lists padded to a common top-k with `topk_len`: only the
    leading slots are read, and splits beyond the last tile come out empty."""
    case = orc.make_csa_case(seed=72, B=3, s_q=1, H=32, n_entries=[40, 700, 129], topk=512, ragged=True)
    topk_len = np.array([[40], [512], [129]], np.int32)
    case.indices[1, 0, 300:] = np.where(np.arange(212) % 2 == 0, -1, case.indices[1, 0, 300:])   # holes inside the prefix
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale,
                                               kv_len=case.kv_len)
    args = gu.csa_to_dev(case)
    for splits in (1, 4, 8):
        st = lib.new_status("cuda")
        out, lse = lib.csa_sparse_decode(**args, topk_len=gu.dev(topk_len), num_splits=splits, status=st)
        torch.cuda.synchronize()
        assert st.cpu().tolist() == [0, 0, 0, 0]
        gu.check_out(gu.out_to_f32(out), want_out, f"topk_len splits={splits}")
        gu.check_lse(lse.cpu().numpy(), want_lse, f"topk_len splits={splits}")


def test_reference_entry_point_split_path(lib):
    """hca_decode_fwd with a context long enough that the library splits it
    (B=1 leaves most SMs idle otherwise) and merges inside the same call."""
    c = orc.make_ref_layout_case(seed=73, B=1, H=128, M_cur=1920, swa_len=128)
    want, _ = orc.hca_decode_ref_layout(c.Q, c.Kc, c.Kc_s, c.Kc_rope, c.Kswa, c.Kswa_s, c.Kswa_rope, c.sink, c.sm_scale)
    d = gu.dev
    assert lib.plan_splits(1, 128, 2048) > 1
    O = lib.hca_decode_fwd(d(c.Q, torch.bfloat16), d(c.Kc), d(c.Kc_s), d(c.Kc_rope, torch.bfloat16),
                           d(c.Kswa), d(c.Kswa_s), d(c.Kswa_rope, torch.bfloat16), d(c.sink), c.sm_scale,
                           M_cur=1920, swa_len=128)
    torch.cuda.synchronize()
    gu.check_out(gu.out_to_f32(O), want, "hca_decode_fwd split")


@pytest.mark.parametrize("page_size", [16, 64])
def test_packed_pages_decode_vs_reference_outputs(lib, page_size):
    """Packed cache pages read in place: the reference-layout golden cases repacked into
    pages give the reference's outputs; per-request lengths give the oracle's."""
    for name in ("ref_layout", "ref_layout_ragged"):
        z, kw = golden(name)
        c = orc.make_ref_layout_case(**kw)
        B, H = c.Q.shape[:2]
        rng = np.random.default_rng(9)
        kv_pages, bt = orc.pack_ref_pages(c.Kc, c.Kc_s, c.Kc_rope, page_size, rng)
        sw_pages, sbt = orc.pack_ref_pages(c.Kswa, c.Kswa_s, c.Kswa_rope, page_size, rng)
        d = lambda a: gu.dev(a)
        q = gu.dev(c.Q, torch.bfloat16)
        status = lib.new_status(q.device)
        full = (np.full(B, c.Kc.shape[1], np.int32), np.full(B, c.Kswa.shape[1], np.int32))
        ragged = (np.array([c.Kc.shape[1] - 7, 1][:B], np.int32), np.array([0, c.Kswa.shape[1]][:B], np.int32))
        for m_cur, swa in (full, ragged):
            for splits in (1, 2):
                out, lse = lib.hca_packed_decode(q, d(kv_pages), d(bt), d(m_cur), d(sw_pages), d(sbt), d(swa), c.sm_scale,
                                                 page_size=page_size, attn_sink=gu.dev(c.sink), num_splits=splits, status=status)
                torch.cuda.synchronize()
                assert status.cpu().tolist() == [0, 0, 0, 0]
                want, want_lse = orc.hca_decode_packed_pages(c.Q, kv_pages, bt, m_cur, sw_pages, sbt, swa, c.sink, c.sm_scale, page_size)
                gu.check_out(gu.out_to_f32(out), want, f"{name} ps={page_size} splits={splits}")
                gu.check_lse(lse.cpu().numpy(), want_lse, f"{name} ps={page_size}")
                if m_cur is full[0]:
                    gu.check_out(gu.out_to_f32(out), z["out_fp8_dequant"], f"{name} vs reference output")


def test_packed_pages_decode_bad_tables_and_arguments(lib):
    """A block-table value outside the pool drops those tokens instead of reading them; bad
    shapes are refused on the host."""
    c = orc.make_ref_layout_case(seed=81, B=2, H=16, M_cur=128, swa_len=16)
    rng = np.random.default_rng(3)
    kv_pages, bt = orc.pack_ref_pages(c.Kc, c.Kc_s, c.Kc_rope, 64, rng)
    sw_pages, sbt = orc.pack_ref_pages(c.Kswa, c.Kswa_s, c.Kswa_rope, 64, rng)
    q = gu.dev(c.Q, torch.bfloat16)
    m_cur, swa = np.array([128, 128], np.int32), np.array([16, 16], np.int32)
    bad = bt.copy()
    bad[1, 1] = kv_pages.shape[0] + 5          # request 1 loses tokens 64..127
    out, lse = lib.hca_packed_decode(q, gu.dev(kv_pages), gu.dev(bad), gu.dev(m_cur), gu.dev(sw_pages), gu.dev(sbt), gu.dev(swa),
                                     c.sm_scale, num_splits=1)
    torch.cuda.synchronize()
    want, _ = orc.hca_decode_packed_pages(c.Q, kv_pages, bt, np.array([128, 64], np.int32), sw_pages, sbt, swa, None, c.sm_scale, 64)
    gu.check_out(gu.out_to_f32(out), want, "bad table entry")
    with pytest.raises(ValueError):
        lib.hca_packed_decode(q, gu.dev(kv_pages)[:, :100].contiguous(), gu.dev(bt), gu.dev(m_cur), gu.dev(sw_pages), gu.dev(sbt),
                              gu.dev(swa), c.sm_scale)
    with pytest.raises(ValueError):
        lib.hca_packed_decode(q, gu.dev(kv_pages), gu.dev(bt), gu.dev(m_cur), gu.dev(sw_pages), gu.dev(sbt), gu.dev(swa), c.sm_scale,
                              page_size=48)


@pytest.mark.parametrize("splits", [1, 3])
def test_csa_with_attention_sink(lib, splits):
    """The sink option of the CSA entry point (the reference applies the sink in its dense
    softmax, bench/bench/reference.py:294-303, and in its merge, hca/sm100/combine.cu:83-89):
    it enters the denominator only, unsplit and split alike; the LSE stays sink-free."""
    case = orc.make_csa_case(seed=91, B=2, s_q=2, H=32, n_entries=[400, 77], topk=256, ragged=True)
    sink = np.random.default_rng(91).standard_normal(32).astype(np.float32)
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale,
                                               kv_len=case.kv_len, sink=sink)
    out, lse = run_csa(lib, case, num_splits=splits, attn_sink=gu.dev(sink))
    gu.check_out(out, want_out, f"csa sink splits={splits}")
    gu.check_lse(lse, want_lse, f"csa sink splits={splits}")
    no_sink, _ = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale, kv_len=case.kv_len)
    assert np.abs(gu.bits_to_f32(no_sink) - gu.bits_to_f32(want_out)).max() > 1e-2     # the sink matters in this case


def test_large_and_tiny_magnitudes_stay_finite_and_close(lib):
    """The packed layout runs through FP16 operands: entries up to a few tens of thousands and
    blocks of very small values must neither overflow nor lose the result.  Entry magnitudes vary
    by page (x 1e-4 ... x 1e4); tolerance relative to the largest output value."""
    rng = np.random.default_rng(93)
    B, H, n_ent, W = 2, 32, 300, 128
    pages = 5
    mag = np.array([1e-4, 1.0, 300.0, 1e4, 3.0], np.float32)     # largest entries ~4.5e4, inside the 65504 limit
    lat = rng.standard_normal((B * pages, orc.PAGE_ENTRIES, orc.D_LATENT), dtype=np.float32) * np.tile(mag, B)[:, None, None]
    rope = rng.standard_normal((B * pages, orc.PAGE_ENTRIES, orc.D_ROPE), dtype=np.float32)
    pool = orc.pack_entries(lat, rope)
    bt = rng.permutation(B * pages).astype(np.int32).reshape(B, pages)
    win = orc.pack_entries(rng.standard_normal((B, W, orc.D_LATENT), dtype=np.float32) * np.float32(50),
                           rng.standard_normal((B, W, orc.D_ROPE), dtype=np.float32))
    q = orc.bf16_round(rng.standard_normal((B, 1, H, orc.D_QK), dtype=np.float32) * np.float32(0.05))
    kv_len = np.full((B, 1), n_ent, np.int32)
    win_len = np.full((B, 1), 77, np.int32)
    sm = orc.D_QK ** -0.5
    want_out, want_lse = orc.hca_dense_decode(q, pool, bt, kv_len, win, win_len, sm)
    out, lse = lib.hca_dense_decode(gu.dev(q, torch.bfloat16), gu.dev(pool), gu.dev(bt), gu.dev(kv_len), gu.dev(win),
                                    gu.dev(win_len), sm, num_splits=1)
    torch.cuda.synchronize()
    got = gu.out_to_f32(out)
    want = gu.bits_to_f32(want_out)
    assert np.isfinite(got).all() and np.isfinite(lse.cpu().numpy()).all()
    scale = np.abs(want).max()
    assert scale > 100          # the large entries do carry weight here
    assert np.abs(got - want).max() <= 2e-2 * scale
    assert np.abs(got - want).mean() <= 2e-3 * scale
    gu.check_lse(lse.cpu().numpy(), want_lse, "large magnitudes")


def test_entry_points_replay_from_a_cuda_graph(lib):
    """The entry points only enqueue kernels on the caller's stream (tensor maps travel by value
    as kernel parameters), so they can be captured into a CUDA graph and replayed, which is how
    the reference's graph candidate calls hca_decode_fwd
    (bench/bench/candidates/hca_custom_decode_graph.py:49-53).  Replays after the inputs changed
    in place give the new inputs' results."""
    z, kw = golden("ref_layout")
    c = orc.make_ref_layout_case(**kw)
    d = gu.dev
    Q = d(c.Q, torch.bfloat16)
    args = (Q, d(c.Kc), d(c.Kc_s), d(c.Kc_rope, torch.bfloat16), d(c.Kswa), d(c.Kswa_s), d(c.Kswa_rope, torch.bfloat16),
            d(c.sink), c.sm_scale)
    B, n_h, dq = Q.shape
    O = torch.empty(B, n_h, dq, dtype=torch.bfloat16, device="cuda")
    S = (kw["M_cur"] + kw["swa_len"]) // 128
    pO = torch.empty(max(S, 1), B, n_h, dq, dtype=torch.float32, device="cuda")
    pl = torch.empty(max(S, 1), B, n_h, dtype=torch.float32, device="cuda")
    case = orc.make_csa_case(seed=31, B=2, s_q=1, H=32, n_entries=[400, 130], topk=128, ragged=True)
    cargs = gu.csa_to_dev(case)
    c_out = torch.empty(2, 1, 32, 512, dtype=torch.bfloat16, device="cuda")
    c_lse = torch.empty(2, 1, 32, dtype=torch.float32, device="cuda")
    ws = lib.alloc_workspace(2, 32, 2, "cuda")

    def both():
        lib.hca_decode_fwd(*args, M_cur=kw["M_cur"], swa_len=kw["swa_len"], O=O, partial_O=pO, partial_lse=pl)
        lib.csa_sparse_decode(**cargs, num_splits=2, out=c_out, lse=c_lse, workspace=ws)

    both()                                   # one eager call first: per-device kernel attributes are set lazily
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        both()
    O.zero_();  c_out.zero_()
    g.replay()
    torch.cuda.synchronize()
    gu.check_out(gu.out_to_f32(O), z["out_fp8_dequant"], "graph replay, reference entry point")
    want_out, _ = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale, kv_len=case.kv_len)
    gu.check_out(gu.out_to_f32(c_out), want_out, "graph replay, CSA")
    # new queries in the same buffers, same graph
    q2 = orc.bf16_round(np.random.default_rng(5).standard_normal(case.q.shape, dtype=np.float32))
    cargs["q"].copy_(gu.dev(q2, torch.bfloat16))
    g.replay()
    torch.cuda.synchronize()
    want2, _ = orc.csa_sparse_decode(q2, case.pool, case.block_table, case.indices, case.sm_scale, kv_len=case.kv_len)
    gu.check_out(gu.out_to_f32(c_out), want2, "graph replay with new queries")
