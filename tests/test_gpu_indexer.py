"""GPU parity of the CSA indexer (FP8 scoring on the tensor cores + top-k), through the
C ABI, against the CPU oracle and the committed reference selection.  Run with `-m gpu`."""
import ast
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import dsv4_oracle as orc  # noqa: E402
from tests import gpu_util as gu  # noqa: E402
from tests.test_oracle import indexer_inputs  # noqa: E402

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as d
    return d


def run(lib, c, pages, bt, qw, n_vis, k):
    status = lib.new_status("cuda")
    idx, scores = lib.indexer_topk(gu.dev(c.q_fp8), gu.dev(qw), gu.dev(pages), gu.dev(bt), gu.dev(n_vis), k, status=status)
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0], f"a bounded wait gave up: {status.cpu().tolist()}"
    return idx.cpu().numpy(), scores.cpu().numpy()


def check_selection(idx, gpu_scores, want_scores, n_vis, k):
    """Scores within FP32 accumulation-order noise of the oracle's; the selection has the right
    size, no repeats, only visible entries, and no entry left out scores more than the noise
    above one that was taken."""
    B, s_q = n_vis.shape
    for b in range(B):
        for t in range(s_q):
            v = int(n_vis[b, t])
            row = b * s_q + t
            want = want_scores[b, t, :v]
            if v:
                tol = 1e-4 * np.abs(want).max() + 1e-6
                assert np.abs(gpu_scores[row, :v] - want).max() <= tol, (b, t)
            got = idx[b, t]
            taken = got[got >= 0]
            assert len(taken) == min(k, v) and (got[len(taken):] == -1).all() if v < k else len(taken) == k
            assert len(np.unique(taken)) == len(taken) and (taken < v).all()
            if v > k:
                left = np.setdiff1d(np.arange(v), taken)
                assert want[left].max() <= want[taken].min() + 2 * tol, (b, t)


def test_indexer_vs_reference_selection(lib):
    z = np.load(GOLD / "indexer_topk.npz")
    kw = ast.literal_eval(str(z["kwargs"]))
    c = orc.make_indexer_case(**{k: v for k, v in kw.items() if k not in ("m", "top_k", "tokens")})
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(2))
    idx, scores = run(lib, c, pages, bt, qw, z["n_vis"], kw["top_k"])
    want = orc.indexer_scores(c.q_fp8, qw, pages, bt, z["n_vis"])
    check_selection(idx, scores, want, z["n_vis"], kw["top_k"])
    for b in range(idx.shape[0]):
        for t in range(idx.shape[1]):
            assert np.array_equal(np.sort(idx[b, t]), np.sort(z["sel"][b, t])), (b, t)


@pytest.mark.parametrize("s_q,n,k,n_vis", [
    (1, 64, 16, None), (2, 1000, 128, [[1000, 937], [5, 0], [129, 128]]), (1, 5000, 512, [[5000], [4097]]),
    (2, 333, 512, [[333, 200]]),
])
def test_indexer_vs_oracle(lib, s_q, n, k, n_vis):
    B = 1 if n_vis is None else len(n_vis)
    c = orc.make_indexer_case(seed=100 + n, B=B, s_q=s_q, n=n, n_vis=n_vis)
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(3))
    idx, scores = run(lib, c, pages, bt, qw, c.n_vis, k)
    want = orc.indexer_scores(c.q_fp8, qw, pages, bt, c.n_vis)
    check_selection(idx, scores, want, c.n_vis, k)


def test_indexer_feeds_the_sparse_decode(lib):
    """The index list the indexer writes (-1 padded, unordered) is what the CSA decode entry
    point takes: same result as the oracle's decode over the oracle's selection."""
    case = orc.make_csa_case(seed=7, B=2, s_q=1, H=16, n_entries=[300, 90], topk=64, ragged=True)
    c = orc.make_indexer_case(seed=8, B=2, s_q=1, n=300, n_vis=[[300], [90]])
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(4))
    idx, _ = run(lib, c, pages, bt, qw, c.n_vis, 64)
    want_sel = orc.indexer_topk(orc.indexer_scores(c.q_fp8, qw, pages, bt, c.n_vis), c.n_vis, 64)
    for b in range(2):
        assert np.array_equal(np.sort(idx[b, 0][idx[b, 0] >= 0]), want_sel[b][0])
    args = gu.csa_to_dev(case)
    args["indices"] = gu.dev(idx)
    out, lse = lib.csa_sparse_decode(**args)
    torch.cuda.synchronize()
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, idx, case.sm_scale, kv_len=case.kv_len)
    gu.check_out(gu.out_to_f32(out), want_out, "decode over the indexer's selection")
    gu.check_lse(lse.cpu().numpy(), want_lse, "decode over the indexer's selection")


def test_indexer_invalid_arguments(lib):
    c = orc.make_indexer_case(seed=9, B=1, s_q=1, n=64)
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(5))
    with pytest.raises(ValueError):
        lib.indexer_topk(gu.dev(c.q_fp8)[:, :, :32].contiguous(), gu.dev(qw), gu.dev(pages), gu.dev(bt), gu.dev(c.n_vis), 8)
    with pytest.raises(ValueError):
        lib.indexer_topk(gu.dev(c.q_fp8), gu.dev(qw), gu.dev(pages)[:, :8000].contiguous(), gu.dev(bt), gu.dev(c.n_vis), 8)
    with pytest.raises(ValueError):
        lib.indexer_topk(gu.dev(c.q_fp8), gu.dev(qw), gu.dev(pages), gu.dev(bt), gu.dev(c.n_vis), 0)


def test_indexer_many_rows_single_block_per_row(lib):
    """With more rows than half the SMs the selection runs one block per row (fewer rows share a
    row between a cluster pair of blocks): both paths must agree with the oracle."""
    B = 80
    rng = np.random.default_rng(17)
    n_vis = rng.integers(1, 400, size=(B, 1)).astype(np.int32)
    n_vis[0, 0], n_vis[1, 0] = 400, 33
    c = orc.make_indexer_case(seed=117, B=B, s_q=1, n=400, n_vis=n_vis)
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(6))
    idx, scores = run(lib, c, pages, bt, qw, c.n_vis, 32)
    want = orc.indexer_scores(c.q_fp8, qw, pages, bt, c.n_vis)
    check_selection(idx, scores, want, c.n_vis, 32)


def test_topk_with_many_equal_scores(lib):
    """All keys equal: every score of a row is the same, the threshold bin holds the whole row and
    the in-place fallback of the selection runs; any k distinct visible entries are a valid answer."""
    c = orc.make_indexer_case(seed=118, B=2, s_q=1, n=6000)
    c.K[:] = c.K[:, :1]                       # identical keys per request
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(7))
    idx, scores = run(lib, c, pages, bt, qw, c.n_vis, 100)
    for b in range(2):
        taken = idx[b, 0]
        assert (taken >= 0).all() and (taken < 6000).all() and len(np.unique(taken)) == 100
        assert np.ptp(scores[b, :6000]) <= 1e-5 * np.abs(scores[b, :6000]).max() + 1e-6


def test_indexer_bounded_wait_runs_out_and_kernel_returns(lib):
    """With the limit of the barrier waits set to 200 us and one "accumulator full" signal withheld in every
    block of the scoring kernel, the launch returns (no trap, no fault, no hang) with the status naming the
    wait, and the next launch is an ordinary one."""
    c = orc.make_indexer_case(seed=171, B=2, s_q=1, n=1500, n_vis=None)
    pages, bt, qw = indexer_inputs(c, np.random.default_rng(5))
    status = lib.new_status("cuda")
    lib.LIB.dsv4_debug_set_wait(200_000, 0)
    try:
        lib.indexer_topk(gu.dev(c.q_fp8), gu.dev(qw), gu.dev(pages), gu.dev(bt), gu.dev(c.n_vis), 256, status=status)
        torch.cuda.synchronize()
    finally:
        lib.LIB.dsv4_debug_set_wait(0, -1)
    code, block, role, tile = status.cpu().tolist()
    assert code == 32, f"expected the indexer's wait code, got {status.cpu().tolist()}"
    assert role in (0, 1, 2)
    idx, scores = run(lib, c, pages, bt, qw, c.n_vis, 256)
    check_selection(idx, scores, orc.indexer_scores(c.q_fp8, qw, pages, bt, c.n_vis), c.n_vis, 256)
