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


def test_noalloc_entry_point_at_exactly_its_limit():
    """16 splits x 8 rows x 128 heads x 512 values = 8 Mi floats: the whole built-in array, accepted and correct;
    one row more is refused."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import dsv4_attn_b200 as lib
    case = orc.make_csa_case(seed=54, B=8, s_q=1, H=128, n_entries=2048, topk=2048)
    args = gu.csa_to_dev(case)
    assert 16 * 8 * 128 * 512 == 8 << 20
    out = torch.full((8, 1, 128, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((8, 1, 128), float("nan"), dtype=torch.float32, device="cuda")
    st = lib.new_status("cuda")
    lib.csa_sparse_decode_noalloc(**args, out=out, lse=lse, num_splits=16, status=st)
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, 0, 0, 0]
    o_bits, o_lse = orc.csa_sparse_decode(case.q, case.pool, case.block_table, case.indices, case.sm_scale, kv_len=case.kv_len)
    gu.check_out(out.float().cpu().numpy(), o_bits, "noalloc at the limit")
    gu.check_lse(lse.cpu().numpy(), o_lse, "noalloc at the limit")
    case9 = orc.make_csa_case(seed=55, B=9, s_q=1, H=128, n_entries=2048, topk=2048)
    out9 = torch.empty(9, 1, 128, 512, dtype=torch.bfloat16, device="cuda")
    lse9 = torch.empty(9, 1, 128, dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError, match="exceed the built-in scratch"):
        lib.csa_sparse_decode_noalloc(**gu.csa_to_dev(case9), out=out9, lse=lse9, num_splits=16)


def test_noalloc_entry_point_names_a_rejected_argument():
    """A parameter block the library refuses comes back as cudaErrorInvalidValue with "invalid argument" as the
    thread's last error, and nothing is launched."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ctypes as C
    import dsv4_attn_b200 as lib
    from dsv4_attn_b200 import _lib
    case = orc.make_csa_case(seed=56, B=2, s_q=1, H=128, n_entries=512, topk=256)
    a = gu.csa_to_dev(case)
    out = torch.empty(2, 1, 128, 512, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(2, 1, 128, dtype=torch.float32, device="cuda")
    ptr = lambda t: t.data_ptr()
    good = dict(B=2, s_q=1, H=128, topk=256, max_pages=a["block_table"].shape[1], num_splits=2, sm_scale=float(case.sm_scale),
                num_pages=a["kv_pool"].shape[0], q=ptr(a["q"]), kv_pool=ptr(a["kv_pool"]), block_table=ptr(a["block_table"]),
                indices=ptr(a["indices"]), out=ptr(out), lse=ptr(lse))
    for bad in (dict(H=0), dict(topk=0), dict(num_splits=0), dict(q=None), dict(num_pages=0)):
        p = _lib.CsaSparseDecodeParams(**{**good, **bad})
        rc = _lib.LIB.dsv4_csa_sparse_decode_fwd_noalloc(C.byref(p), None)
        assert rc == 1, bad                                     # cudaErrorInvalidValue
        assert _lib.LIB.dsv4_attn_last_error().decode() == "invalid argument", bad
    assert _lib.LIB.dsv4_csa_sparse_decode_fwd_noalloc(None, None) == 1
    assert _lib.LIB.dsv4_attn_last_error().decode() == "null parameter block"
    p = _lib.CsaSparseDecodeParams(**good)
    assert _lib.LIB.dsv4_csa_sparse_decode_fwd_noalloc(C.byref(p), None) == 0
    assert _lib.LIB.dsv4_attn_last_error().decode() == ""
    torch.cuda.synchronize()
