"""GPU tests of the split-KV scheduler: the planner kernel against its host twin, and the decode entry
points walking a plan (resident blocks, several items per block, rows cut over blocks, per-row split
counts in the merge) against the oracle.  Run with `-m gpu` on a B200."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import dsv4_oracle as orc  # noqa: E402
from tests import gpu_util as gu  # noqa: E402
from tests.test_sched_host import check_cover, layout, PAIRS_OFF  # noqa: E402


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as d
    return d


def device_plan_view(plan, sms):
    buf = plan.sched.cpu().numpy()
    hgs = (plan.H + 127) // 128
    n_units = plan.B * plan.s_q * hgs
    ns, slot, items = layout(n_units)
    n_items, n_slots, over, quota = buf[:4].tolist()
    assert over == 0
    pairs = sms // 2
    return dict(pair_begin=buf[PAIRS_OFF:PAIRS_OFF + pairs + 1], nsplits=buf[ns:ns + n_units], slot=buf[slot:slot + n_units],
                items=buf[items:items + 8 * n_items].reshape(n_items, 8), n_slots=n_slots, quota=quota,
                slot_cap=plan.partial_o.numel() * 4 // (128 * 512 * 2), hgs=hgs, pairs=pairs)


def test_planner_kernel_covers_every_row_once(lib):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rng = np.random.default_rng(5)
    kv = rng.integers(0, 2000, size=(300, 1)).astype(np.int32)
    win = rng.integers(0, 129, size=(300, 1)).astype(np.int32)
    kv[7] = 0;  win[7] = 0
    plan = lib.plan_hca(300, 1, 128, gu.dev(kv), gu.dev(win))
    torch.cuda.synchronize()
    view = device_plan_view(plan, sms)
    cost = check_cover(view, (kv + win).reshape(-1).tolist())
    assert cost.max() <= view["quota"] + 2 * 48 + 2 * 32
    plan8 = lib.plan_csa(5, 2, 128, 2048, num_splits=8)
    torch.cuda.synchronize()
    v8 = device_plan_view(plan8, sms)
    check_cover(v8, [2048] * 10)
    # 80 pieces on 74 pairs: where two consecutive pieces of a unit fall to one pair they run as one item
    assert (v8["nsplits"] <= 8).all() and (v8["nsplits"] >= 6).all()


def run(lib, kind, case, plan):
    st = lib.new_status("cuda")
    if kind == "csa":
        out, lse = lib.csa_sparse_decode(status=st, plan=plan, **gu.csa_to_dev(case))
    else:
        out, lse = lib.hca_dense_decode(status=st, plan=plan, **gu.hca_to_dev(case))
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0], f"status {st.cpu().tolist()}"
    return gu.out_to_f32(out), lse.cpu().numpy()


@pytest.mark.parametrize("splits", [0, 1, 3, 8])
def test_csa_with_plan(lib, splits):
    case = orc.make_csa_case(seed=31, B=5, s_q=2, H=128, n_entries=[700, 1500, 90, 64, 2500], topk=1024, ragged=True)
    case.indices[3, 1, :] = -1
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale, kv_len=case.kv_len)
    plan = lib.plan_csa(5, 2, 128, 1024, kv_len=gu.dev(case.kv_len), num_splits=splits)
    out, lse = run(lib, "csa", case, plan)
    gu.check_out(out, want_out, f"csa plan splits={splits}")
    gu.check_lse(lse, want_lse, f"csa plan splits={splits}")
    if splits == 0:
        assert plan.info()[1] > 0      # few rows on many SMs: rows were cut


@pytest.mark.parametrize("splits", [0, 4])
def test_hca_with_plan_sink_and_empty_rows(lib, splits):
    case = orc.make_hca_case(seed=32, B=6, s_q=2, H=128, kv_len=[782, 333, 0, 5, 1900, 64], win_len=[128, 40, 0, 1, 128, 0],
                             with_sink=True)
    want_out, want_lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len, case.win, case.win_len,
                                              case.sm_scale, sink=case.sink)
    plan = lib.plan_hca(6, 2, 128, gu.dev(case.kv_len), gu.dev(case.win_len), num_splits=splits)
    out, lse = run(lib, "hca", case, plan)
    gu.check_out(out, want_out, f"hca plan splits={splits}")
    gu.check_lse(lse, want_lse, f"hca plan splits={splits}")


def test_many_short_rows_share_blocks(lib):
    """More rows than block pairs: every resident block works through several items, most of them whole rows
    written out directly, and the set-up of each next item overlaps the tail of the current one."""
    rng = np.random.default_rng(9)
    B = 200
    kv = rng.integers(1, 400, size=B).tolist()
    win = rng.integers(0, 129, size=B).tolist()
    case = orc.make_hca_case(seed=33, B=B, s_q=1, H=128, kv_len=kv, win_len=win)
    plan = lib.plan_hca(B, 1, 128, gu.dev(case.kv_len), gu.dev(case.win_len))
    out, lse = run(lib, "hca", case, plan)
    # the numpy oracle on 24 rows (first, last, and a spread); every row against the plain-SIMT kernel on the device
    rows = sorted({0, B - 1, *np.linspace(0, B - 1, 22).astype(int).tolist()})
    sub = lambda a: a[rows]
    want_out, want_lse = orc.hca_dense_decode(sub(case.q), case.pool, sub(case.block_table), sub(case.kv_len), sub(case.win),
                                              sub(case.win_len), case.sm_scale)
    gu.check_out(out[rows], want_out, "many short rows")
    gu.check_lse(lse[rows], want_lse, "many short rows")
    o2, l2 = lib.hca_dense_decode(impl="simt", **gu.hca_to_dev(case))
    torch.cuda.synchronize()
    assert np.abs(out - gu.out_to_f32(o2)).max() <= 2e-2
    np.testing.assert_allclose(lse, l2.cpu().numpy(), rtol=1e-3, atol=1e-3)


def test_two_head_groups_with_plan(lib):
    case = orc.make_csa_case(seed=34, B=3, s_q=1, H=192, n_entries=[300, 1000, 129], topk=512, ragged=True)
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale, kv_len=case.kv_len)
    plan = lib.plan_csa(3, 1, 192, 512, kv_len=gu.dev(case.kv_len))
    out, lse = run(lib, "csa", case, plan)
    gu.check_out(out, want_out, "H=192 plan")
    gu.check_lse(lse, want_lse, "H=192 plan")


def test_plan_reuse_and_graph_replay(lib):
    """One plan, two 'layers' (different queries and caches of the same lengths), planner and both decode calls
    captured into one CUDA graph and replayed."""
    a = orc.make_hca_case(seed=35, B=4, s_q=1, H=128, kv_len=[500, 100, 900, 30], win_len=[128, 128, 16, 2])
    b = orc.make_hca_case(seed=36, B=4, s_q=1, H=128, kv_len=[500, 100, 900, 30], win_len=[128, 128, 16, 2])
    da, db = gu.hca_to_dev(a), gu.hca_to_dev(b)
    plan = lib.plan_hca(4, 1, 128, da["kv_len"], da["win_len"])
    oa = torch.empty(4, 1, 128, 512, dtype=torch.bfloat16, device="cuda");  la = torch.empty(4, 1, 128, device="cuda")
    ob = torch.empty_like(oa);  lb = torch.empty_like(la)
    st = lib.new_status("cuda")
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        lib.hca_dense_decode(plan=plan, out=oa, lse=la, status=st, **da)      # warm-up outside the capture
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            plan.remake()
            lib.hca_dense_decode(plan=plan, out=oa, lse=la, status=st, **da)
            lib.hca_dense_decode(plan=plan, out=ob, lse=lb, status=st, **db)
        oa.zero_();  ob.zero_()
        g.replay()
        s.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0]
    for case, o, l in ((a, oa, la), (b, ob, lb)):
        want_out, want_lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len, case.win, case.win_len, case.sm_scale)
        gu.check_out(gu.out_to_f32(o), want_out, "graph replay with plan")
        gu.check_lse(l.cpu().numpy(), want_lse, "graph replay with plan")


def test_plan_for_another_batch_is_rejected(lib):
    case = orc.make_csa_case(seed=37, B=2, s_q=1, H=128, n_entries=300, topk=256)
    plan = lib.plan_csa(3, 1, 128, 256)
    with pytest.raises(ValueError):
        lib.csa_sparse_decode(plan=plan, **gu.csa_to_dev(case))
