"""The entry point that allocates nothing (dsv4_csa_sparse_decode_fwd_noalloc).

It serves hosts that cannot allocate device memory at decode time - an engine
that has given all of HBM to its KV-cache pool, a plug-in that must not touch
its host's allocator - by keeping the split-KV partials in a fixed array inside
the library.  The test calls it through the C ABI twice in a row, on different
inputs, and checks each result against the ordinary entry point (which takes a
caller workspace) with the tolerance of the other parity tests; it also checks
that a request larger than the built-in array is refused.  The file name sorts
last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import dsv4_oracle as orc  # noqa: E402
from tests import gpu_util as gu  # noqa: E402


def test_noalloc_entry_point_matches_workspace_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as lib
    assert lib.LIB.dsv4_noalloc_scratch_bytes() == (8 << 20) * 4 + (8 << 20) // 512 * 4
    for seed, splits in ((51, 4), (52, 3)):                  # two calls in a row share the scratch
        case = orc.make_csa_case(seed=seed, B=2, s_q=2, H=32, n_entries=[900, 300], topk=512, ragged=True)
        args = gu.csa_to_dev(case)
        st = lib.new_status("cuda")
        want_out, want_lse = lib.csa_sparse_decode(**args, num_splits=splits, status=st)
        out = torch.full_like(want_out, float("nan"))
        lse = torch.full_like(want_lse, float("nan"))
        lib.csa_sparse_decode_noalloc(**args, out=out, lse=lse, num_splits=splits, status=st)
        torch.cuda.synchronize()
        assert st.cpu().tolist() == [0, 0, 0, 0]
        a, b = out.float().cpu().numpy(), want_out.float().cpu().numpy()
        assert np.isfinite(a).all()
        assert np.abs(a - b).max() <= gu.OUT_MAX_ABS and np.abs(a - b).mean() <= gu.OUT_MEAN_ABS
        gu.check_lse(lse.cpu().numpy(), want_lse.cpu().numpy(), "noalloc")
        # and against the CPU oracle, like every other parity test
        o_bits, o_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale,
                                              kv_len=case.kv_len)
        gu.check_out(a, o_bits, "noalloc vs oracle")
        gu.check_lse(lse.cpu().numpy(), o_lse, "noalloc vs oracle")
    # one split needs no scratch at all
    lib.csa_sparse_decode_noalloc(**args, out=out, lse=lse, num_splits=1)
    torch.cuda.synchronize()
    gu.check_out(out.float().cpu().numpy(), o_bits, "noalloc, one split")


def test_noalloc_entry_point_refuses_oversized_requests():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as lib
    case = orc.make_csa_case(seed=53, B=5, s_q=1, H=128, n_entries=2048, topk=2048)
    args = gu.csa_to_dev(case)
    out = torch.empty(5, 1, 128, 512, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(5, 1, 128, dtype=torch.float32, device="cuda")
    # 32 splits x 5 rows x 128 heads x 512 = 10 Mi floats > 8 Mi
    with pytest.raises(ValueError, match="exceed the built-in scratch"):
        lib.csa_sparse_decode_noalloc(**args, out=out, lse=lse, num_splits=32)
    lib.csa_sparse_decode_noalloc(**args, out=out, lse=lse, num_splits=16)      # 5 Mi floats fits
    torch.cuda.synchronize()
