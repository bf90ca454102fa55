"""GPU parity at the full shapes of the benchmark configurations (seeded synthetic data, as the
configurations prescribe).  The numpy oracle is too slow for whole batches of this size, so every case
is checked twice: the whole batch against the plain-SIMT kernel on the device (FP32, exact
dequantisation, one block per row and head), and a fixed sample of rows - first, last, longest,
shortest and a spread, at least 16 - against the CPU oracle.  Tolerances: BF16 output max-abs 2e-2 and
mean-abs 2e-3, LSE 1e-3 relative.  Run with `-m gpu` on a B200."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import sample_check as sc  # noqa: E402

OUT_MAX_ABS, OUT_MEAN_ABS, LSE_REL = 2e-2, 2e-3, 1e-3


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as d
    return d


def against_simt(out, lse, ref_out, ref_lse, what):
    err = (out.float() - ref_out.float()).abs()
    assert torch.isfinite(out.float()).all(), f"{what}: non-finite output"
    assert float(err.max()) <= OUT_MAX_ABS, f"{what}: max-abs {float(err.max()):.4g} vs the SIMT kernel"
    assert float(err.mean()) <= OUT_MEAN_ABS, f"{what}: mean-abs {float(err.mean()):.4g} vs the SIMT kernel"
    inf = torch.isneginf(ref_lse)
    assert torch.equal(torch.isneginf(lse), inf), f"{what}: -inf pattern of the LSE differs"
    rel = ((lse - ref_lse).abs() / ref_lse.abs().clamp(min=1.0))[~inf]
    assert rel.numel() == 0 or float(rel.max()) <= LSE_REL, f"{what}: lse rel {float(rel.max()):.4g} vs the SIMT kernel"


def against_oracle(summary, what):
    assert summary["parity_checked_rows"] >= 16
    assert sc.within_tolerance(summary, OUT_MAX_ABS, OUT_MEAN_ABS, LSE_REL), f"{what}: {summary}"
    print(what, summary)


def csa_variants(lib, w, variants, what):
    B, s_q, H, _ = w.q.shape
    topk = w.indices.shape[-1]
    st = lib.new_status("cuda")
    common = dict(kv_len=w.kv_len, topk_len=w.topk_len, status=st)
    ref_out, ref_lse = lib.csa_sparse_decode(w.q, w.kv_pool, w.block_table, w.indices, w.sm_scale, impl="simt", **common)
    rows = sc.pick_rows(w.topk_len, 16)
    for name, kw in variants.items():
        if "plan_splits" in kw:
            kw = dict(plan=lib.plan_csa(B, s_q, H, topk, topk_len=w.topk_len, kv_len=w.kv_len, num_splits=kw["plan_splits"]))
        out, lse = lib.csa_sparse_decode(w.q, w.kv_pool, w.block_table, w.indices, w.sm_scale, **common, **kw)
        torch.cuda.synchronize()
        assert st.cpu().tolist() == [0, 0, 0, 0], f"{what}/{name}: status {st.cpu().tolist()}"
        against_simt(out, lse, ref_out, ref_lse, f"{what}/{name}")
        against_oracle(sc.check_csa_rows(w.q, w.kv_pool, w.block_table, w.indices, w.sm_scale, out, lse, rows,
                                         kv_len=w.kv_len, topk_len=w.topk_len), f"{what}/{name}")


def hca_variants(lib, w, variants, what):
    B, s_q, H, _ = w.q.shape
    st = lib.new_status("cuda")
    args = (w.q, w.kv_pool, w.block_table, w.kv_len, w.win_pool, w.win_len, w.sm_scale)
    ref_out, ref_lse = lib.hca_dense_decode(*args, impl="simt", status=st)
    rows = sc.pick_rows(w.kv_len + w.win_len, 16)
    for name, kw in variants.items():
        if "plan_splits" in kw:
            kw = dict(plan=lib.plan_hca(B, s_q, H, w.kv_len, w.win_len, num_splits=kw["plan_splits"]))
        out, lse = lib.hca_dense_decode(*args, status=st, max_len=w.max_len, **kw)
        torch.cuda.synchronize()
        assert st.cpu().tolist() == [0, 0, 0, 0], f"{what}/{name}: status {st.cpu().tolist()}"
        against_simt(out, lse, ref_out, ref_lse, f"{what}/{name}")
        against_oracle(sc.check_hca_rows(*args, out, lse, rows), f"{what}/{name}")


def test_config1_csa_b64_topk512_paged_no_split(lib):
    from dsv4_attn_b200 import synth
    w = synth.make_csa(101, 64, 1, 128, 768, 512)
    csa_variants(lib, w, {"no split": dict(num_splits=1), "planned": dict(plan_splits=0)}, "config 1")


def test_config1_ragged_contexts_with_padding(lib):
    from dsv4_attn_b200 import synth
    rng = np.random.default_rng(3)
    w = synth.make_csa(102, 64, 1, 128, rng.integers(40, 769, size=64).tolist(), 512)
    assert int((w.indices < 0).sum()) > 0
    csa_variants(lib, w, {"no split": dict(num_splits=1), "planned": dict(plan_splits=0)}, "config 1 ragged")


def test_config2_hca_b64_ctx100k(lib):
    from dsv4_attn_b200 import synth
    w = synth.make_hca(103, 64, 1, 128, 782, 128)
    hca_variants(lib, w, {"no split": dict(num_splits=1), "planned": dict(plan_splits=0), "two pieces": dict(plan_splits=2)},
                 "config 2")


def test_config3_csa_b128_nextn2_topk2048_ctx100k(lib):
    """B=128, two query tokens per request (the second sees one entry more than the first), 25,000 entries
    behind 391-page block tables, top-k 2048: with the 8 splits the configuration names (static grid and
    planned), with the planner's own choice, and unsplit."""
    from dsv4_attn_b200 import synth
    w = synth.make_csa(104, 128, 2, 128, 25000, 2048)
    assert w.block_table.shape[1] == 391 and int(w.kv_len[0, 0]) + 1 == int(w.kv_len[0, 1])
    csa_variants(lib, w, {"8 splits": dict(num_splits=8), "8 planned pieces": dict(plan_splits=8),
                          "planned": dict(plan_splits=0), "no split": dict(num_splits=1)}, "config 3")


def test_config4_mixed_1024_requests_both_layers(lib):
    from dsv4_attn_b200 import synth
    ctx = synth.lognormal_contexts(1024, seed=0)
    csa, hca = synth.make_mixed(105, ctx)
    csa_variants(lib, csa, {"no split": dict(num_splits=1), "planned": dict(plan_splits=0)}, "config 4 CSA layer")
    hca_variants(lib, hca, {"no split": dict(num_splits=1), "planned": dict(plan_splits=0)}, "config 4 HCA layer")
