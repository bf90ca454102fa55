"""Randomised shapes for the two decode entry points against the CPU oracle: odd head counts,
several query tokens, ragged lengths, list lengths that are no multiple of the tile, splits that
leave empty parts, with and without sink.  Run with `-m gpu` on a B200."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import dsv4_oracle as orc  # noqa: E402
from tests import gpu_util as gu  # noqa: E402


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as d
    return d


@pytest.mark.parametrize("seed", range(10))
def test_csa_random_shapes(lib, seed):
    rng = np.random.default_rng(1000 + seed)
    B, s_q = int(rng.integers(1, 5)), int(rng.integers(1, 4))
    H = int(rng.choice([1, 7, 16, 64, 128, 130]))
    n_entries = [int(x) for x in rng.integers(1, 500, size=B)]
    topk = int(rng.integers(1, 300))
    case = orc.make_csa_case(seed=2000 + seed, B=B, s_q=s_q, H=H, n_entries=n_entries, topk=topk, ragged=True)
    sink = rng.standard_normal(H).astype(np.float32) if seed % 2 else None
    splits = int(rng.integers(1, 4))
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale,
                                               kv_len=case.kv_len, sink=sink)
    st = lib.new_status("cuda")
    out, lse = lib.csa_sparse_decode(**gu.csa_to_dev(case), num_splits=splits, status=st,
                                     attn_sink=None if sink is None else gu.dev(sink))
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0]
    what = f"B={B} s_q={s_q} H={H} n={n_entries} topk={topk} splits={splits}"
    gu.check_out(gu.out_to_f32(out), want_out, what)
    gu.check_lse(lse.cpu().numpy(), want_lse, what)


@pytest.mark.parametrize("seed", range(10))
def test_hca_random_shapes(lib, seed):
    rng = np.random.default_rng(3000 + seed)
    B, s_q = int(rng.integers(1, 5)), int(rng.integers(1, 3))
    H = int(rng.choice([1, 5, 32, 64, 128, 200]))
    kv_len = [int(x) for x in rng.integers(0, 700, size=B)]
    win_len = [int(x) for x in rng.integers(s_q - 1, 129, size=B)]
    case = orc.make_hca_case(seed=4000 + seed, B=B, s_q=s_q, H=H, kv_len=kv_len, win_len=win_len, with_sink=bool(seed % 2))
    splits = int(rng.integers(1, 5))
    want_out, want_lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len, case.win, case.win_len,
                                              case.sm_scale, sink=case.sink)
    st = lib.new_status("cuda")
    out, lse = lib.hca_dense_decode(**gu.hca_to_dev(case), num_splits=splits, status=st)
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0]
    what = f"B={B} s_q={s_q} H={H} kv={kv_len} win={win_len} splits={splits}"
    gu.check_out(gu.out_to_f32(out), want_out, what)
    gu.check_lse(lse.cpu().numpy(), want_lse, what)
