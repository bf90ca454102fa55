"""GPU tests of the two error paths of the decode kernel, both driven from the host: (1) a bounded wait
that runs out (the loaders are told to withhold one tile's hand-over, the wait limit is set to a fraction
of a millisecond): the kernel must return, name the wait in `status`, and leave the device usable;
(2) indices, lengths and block-table values that point outside the cache: such entries are left out of
the softmax, never read, and reported with status code 7.  Nothing here faults or hangs the GPU."""
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


@pytest.mark.parametrize("with_plan", [False, True])
def test_bounded_wait_runs_out_and_kernel_returns(lib, with_plan):
    case = orc.make_hca_case(seed=61, B=2, s_q=1, H=128, kv_len=[300, 200], win_len=[128, 64])
    args = gu.hca_to_dev(case)
    plan = lib.plan_hca(2, 1, 128, args["kv_len"], args["win_len"]) if with_plan else None
    st = lib.new_status("cuda")
    # 200 us; one tile of every block is never handed over (with a plan the two short rows are cut over all
    # SMs, a tile or two per block: the first one is withheld)
    lib.LIB.dsv4_debug_set_wait(200_000, 0 if with_plan else 1)
    try:
        lib.hca_dense_decode(status=st, plan=plan, num_splits=None if with_plan else 1, **args)
        torch.cuda.synchronize()                    # returns: no trap, no fault, no hang
    finally:
        lib.LIB.dsv4_debug_set_wait(0, -1)
    code, block, role, tile = st.cpu().tolist()
    assert code in (1, 2, 3, 4, 5, 8), f"expected a wait code, got {code}"
    assert role in (0, 1, 2, 3, 4) and tile >= -1
    # the next launch is an ordinary one
    st.zero_()
    out, lse = lib.hca_dense_decode(status=st, plan=plan, num_splits=None if with_plan else 1, **args)
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0]
    want_out, want_lse = orc.hca_dense_decode(case.q, case.pool, case.block_table, case.kv_len, case.win, case.win_len, case.sm_scale)
    gu.check_out(gu.out_to_f32(out), want_out, "after a timed-out launch")
    gu.check_lse(lse.cpu().numpy(), want_lse, "after a timed-out launch")


def test_csa_out_of_range_indices_and_pages_are_left_out(lib):
    case = orc.make_csa_case(seed=62, B=2, s_q=1, H=64, n_entries=[400, 400], topk=256)
    max_pages = case.block_table.shape[1]
    idx = case.indices.copy()
    idx[0, 0, 5] = max_pages * 64 + 3          # beyond the block table
    idx[0, 0, 9] = 2_000_000_000               # far beyond
    bt = case.block_table.copy()
    bad_page_slot = int(idx[1, 0, 0]) >> 6
    bt[1, bad_page_slot] = case.pool.shape[0] + 7       # a table value outside the pool
    # what remains: the same lists with those entries padded out
    ref_idx = idx.copy()
    ref_idx[0, 0, 5] = -1;  ref_idx[0, 0, 9] = -1
    ref_idx[1, 0][(ref_idx[1, 0] >> 6) == bad_page_slot] = -1
    want_out, want_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, ref_idx, case.sm_scale)
    for impl in ("mma", "simt"):
        st = lib.new_status("cuda")
        out, lse = lib.csa_sparse_decode(gu.dev(case.q, torch.bfloat16), gu.dev(case.pool), gu.dev(bt), gu.dev(idx), case.sm_scale,
                                         num_splits=1, status=st, impl=impl)
        torch.cuda.synchronize()
        if impl == "mma":
            assert st.cpu().tolist()[0] == 7
        gu.check_out(gu.out_to_f32(out), want_out, f"bad indices {impl}")
        gu.check_lse(lse.cpu().numpy(), want_lse, f"bad indices {impl}")


def test_hca_lengths_beyond_the_cache_are_left_out(lib):
    case = orc.make_hca_case(seed=63, B=2, s_q=1, H=64, kv_len=[200, 100], win_len=[50, 128])
    max_pages = case.block_table.shape[1]
    kv = case.kv_len.copy();  win = case.win_len.copy()
    kv[0, 0] = max_pages * 64 + 100            # claims more compressed entries than the block table holds
    win[1, 0] = 128 + 40                       # claims more window rows than the window buffer holds
    args = gu.hca_to_dev(case)
    args["kv_len"] = gu.dev(kv);  args["win_len"] = gu.dev(win)
    st = lib.new_status("cuda")
    out, lse = lib.hca_dense_decode(status=st, num_splits=1, **args)
    torch.cuda.synchronize()
    assert st.cpu().tolist()[0] == 7
    got = gu.out_to_f32(out)
    assert np.isfinite(got).all() and np.isfinite(lse.cpu().numpy()).all()
    # request 1: everything readable was attended to - the real 100 + 128 rows
    ref_win = case.win_len.copy()
    want_out, want_lse = orc.hca_dense_decode(case.q[1:], case.pool, case.block_table[1:], case.kv_len[1:], case.win[1:], ref_win[1:],
                                              case.sm_scale)
    gu.check_out(got[1:], want_out, "window length beyond the buffer")
    gu.check_lse(lse.cpu().numpy()[1:], want_lse, "window length beyond the buffer")
