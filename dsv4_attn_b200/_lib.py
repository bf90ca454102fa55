"""ctypes binding of libdsv4_attn.so (the C ABI declared in include/dsv4_attn.h).

The library is the only compute path: if the shared object is missing the
import of this module raises, there is no fallback."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent


class LibraryNotBuilt(ImportError):
    pass


def library_path() -> Path:
    explicit = os.environ.get("DSV4_ATTN_SO")
    return Path(explicit) if explicit else _HERE / "libdsv4_attn.so"


class CsaSparseDecodeParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("s_q", C.c_int32), ("H", C.c_int32), ("topk", C.c_int32),
        ("max_pages", C.c_int32), ("num_splits", C.c_int32), ("sm_scale", C.c_float),
        ("reserved0", C.c_int32), ("num_pages", C.c_int64),
        ("q", C.c_void_p), ("kv_pool", C.c_void_p), ("block_table", C.c_void_p),
        ("indices", C.c_void_p), ("kv_len", C.c_void_p), ("topk_len", C.c_void_p), ("attn_sink", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p), ("partial_o", C.c_void_p),
        ("partial_lse", C.c_void_p), ("status", C.c_void_p), ("sched", C.c_void_p),
    ]


class HcaDenseDecodeParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("s_q", C.c_int32), ("H", C.c_int32), ("max_pages", C.c_int32),
        ("win_cap", C.c_int32), ("num_splits", C.c_int32), ("sm_scale", C.c_float),
        ("reserved0", C.c_int32), ("num_pages", C.c_int64),
        ("q", C.c_void_p), ("kv_pool", C.c_void_p), ("block_table", C.c_void_p),
        ("kv_len", C.c_void_p), ("win_pool", C.c_void_p), ("win_len", C.c_void_p),
        ("attn_sink", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("partial_o", C.c_void_p), ("partial_lse", C.c_void_p), ("status", C.c_void_p), ("sched", C.c_void_p),
    ]


class PlanParams(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("B", C.c_int32), ("s_q", C.c_int32), ("H", C.c_int32), ("topk", C.c_int32),
        ("num_splits", C.c_int32), ("num_sms", C.c_int32), ("reserved0", C.c_int32),
        ("topk_len", C.c_void_p), ("kv_len", C.c_void_p), ("win_len", C.c_void_p),
        ("sched", C.c_void_p), ("sched_bytes", C.c_int64),
    ]


class CombineParams(C.Structure):
    _fields_ = [
        ("N", C.c_int32), ("H", C.c_int32), ("D", C.c_int32), ("num_splits", C.c_int32),
        ("partial_o", C.c_void_p), ("partial_lse", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("attn_sink", C.c_void_p),
        ("stride_po_split", C.c_int64), ("stride_po_n", C.c_int64), ("stride_po_h", C.c_int64),
        ("stride_pl_split", C.c_int64), ("stride_pl_n", C.c_int64),
        ("stride_out_n", C.c_int64), ("stride_out_h", C.c_int64), ("stride_lse_n", C.c_int64),
    ]


EXPORTS = ("dsv4_attn_version", "dsv4_debug_set_wait", "dsv4_debug_set_flags", "dsv4_attn_plan", "dsv4_attn_plan_host", "dsv4_attn_sched_bytes", "dsv4_csa_sparse_decode_fwd", "dsv4_csa_sparse_decode_simt", "dsv4_csa_sparse_decode_fwd_noalloc",
           "dsv4_noalloc_scratch_bytes", "dsv4_attn_last_error", "dsv4_csa_compress_reduce_fwd",
           "dsv4_hca_dense_decode_fwd", "dsv4_hca_dense_decode_simt", "dsv4_attn_combine", "dsv4_attn_plan_splits",
           "dsv4_attn_workspace_bytes", "hca_decode_fwd", "dsv4_hca_compress_fwd", "dsv4_kv_quantize_insert",
           "dsv4_hca_packed_decode_fwd", "dsv4_rope_norm_fwd", "dsv4_indexer_topk_fwd")


class CsaCompressReduceParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("n", C.c_int32), ("c_out", C.c_int32), ("m", C.c_int32),
        ("C_a", C.c_void_p), ("C_b", C.c_void_p), ("Z_a", C.c_void_p), ("Z_b", C.c_void_p),
        ("B_a", C.c_void_p), ("B_b", C.c_void_p), ("out", C.c_void_p),
        ("stride_C_b", C.c_int64), ("stride_C_n", C.c_int64), ("stride_out_b", C.c_int64),
        ("stride_out_blk", C.c_int64),
    ]


class HcaPackedDecodeParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("page_size", C.c_int32), ("max_pages", C.c_int32),
        ("swa_max_pages", C.c_int32), ("num_splits", C.c_int32), ("sm_scale", C.c_float), ("reserved0", C.c_int32),
        ("num_pages", C.c_int64), ("swa_num_pages", C.c_int64),
        ("q", C.c_void_p), ("kv_pages", C.c_void_p), ("block_table", C.c_void_p), ("m_cur", C.c_void_p),
        ("swa_pages", C.c_void_p), ("swa_block_table", C.c_void_p), ("swa_len", C.c_void_p),
        ("attn_sink", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("partial_o", C.c_void_p), ("partial_lse", C.c_void_p), ("status", C.c_void_p),
    ]


class RopeNormParams(C.Structure):
    _fields_ = [
        ("n_rows", C.c_int64), ("vecs_per_row", C.c_int32), ("c", C.c_int32), ("n_rope", C.c_int32), ("inverse", C.c_int32),
        ("eps", C.c_float), ("theta", C.c_float), ("x", C.c_void_p), ("out", C.c_void_p), ("positions", C.c_void_p),
        ("norm_weight", C.c_void_p),
    ]


class IndexerTopkParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("s_q", C.c_int32), ("max_pages", C.c_int32), ("k", C.c_int32),
        ("num_pages", C.c_int64), ("score_stride", C.c_int64),
        ("q_fp8", C.c_void_p), ("q_weight", C.c_void_p), ("key_pages", C.c_void_p), ("block_table", C.c_void_p),
        ("n_vis", C.c_void_p), ("scores", C.c_void_p), ("out_indices", C.c_void_p), ("status", C.c_void_p),
    ]


class CacheDest(C.Structure):
    _fields_ = [
        ("kv_pool", C.c_void_p), ("block_table", C.c_void_p), ("insert_pos", C.c_void_p),
        ("max_pages", C.c_int32), ("reserved0", C.c_int32), ("num_pages", C.c_int64), ("status", C.c_void_p),
    ]


class HcaCompressParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("n", C.c_int32), ("c", C.c_int32), ("m", C.c_int32),
        ("C", C.c_void_p), ("Z", C.c_void_p), ("bias", C.c_void_p),
        ("stride_b", C.c_int64), ("stride_n", C.c_int64), ("out", C.c_void_p), ("dst", C.POINTER(CacheDest)),
    ]


class KvQuantizeInsertParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("T", C.c_int32), ("rows", C.c_void_p),
        ("stride_b", C.c_int64), ("stride_t", C.c_int64), ("n_rows", C.c_void_p), ("dst", C.POINTER(CacheDest)),
    ]


def _load() -> C.CDLL:
    path = library_path()
    if not path.exists():
        raise LibraryNotBuilt(
            f"{path} not found: build it with `python -m dsv4_attn_b200.build` "
            "(needs nvcc; the library has no CPU or PyTorch fallback)")
    lib = C.CDLL(str(path))
    missing = [n for n in EXPORTS if not hasattr(lib, n)]
    if missing:
        raise LibraryNotBuilt(f"{path} is stale (no symbol {missing[0]}): rebuild with `python -m dsv4_attn_b200.build`")
    P = C.POINTER
    lib.dsv4_attn_version.restype = C.c_int
    lib.dsv4_attn_version.argtypes = []
    for name, st in (("dsv4_csa_sparse_decode_fwd", CsaSparseDecodeParams),
                     ("dsv4_csa_sparse_decode_simt", CsaSparseDecodeParams),
                     ("dsv4_csa_sparse_decode_fwd_noalloc", CsaSparseDecodeParams),
                     ("dsv4_hca_dense_decode_fwd", HcaDenseDecodeParams),
                     ("dsv4_hca_dense_decode_simt", HcaDenseDecodeParams),
                     ("dsv4_csa_compress_reduce_fwd", CsaCompressReduceParams),
                     ("dsv4_hca_compress_fwd", HcaCompressParams),
                     ("dsv4_indexer_topk_fwd", IndexerTopkParams),
                     ("dsv4_rope_norm_fwd", RopeNormParams),
                     ("dsv4_hca_packed_decode_fwd", HcaPackedDecodeParams),
                     ("dsv4_kv_quantize_insert", KvQuantizeInsertParams),
                     ("dsv4_attn_plan", PlanParams),
                     ("dsv4_attn_combine", CombineParams)):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [P(st), C.c_void_p]
    lib.dsv4_debug_set_flags.restype = None
    lib.dsv4_debug_set_flags.argtypes = [C.c_int]
    lib.dsv4_debug_set_wait.restype = None
    lib.dsv4_debug_set_wait.argtypes = [C.c_uint64, C.c_int]
    lib.dsv4_attn_plan_host.restype = C.c_int
    lib.dsv4_attn_plan_host.argtypes = [P(PlanParams)]
    lib.dsv4_attn_sched_bytes.restype = C.c_int64
    lib.dsv4_attn_sched_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, P(C.c_int64), P(C.c_int64)]
    lib.dsv4_noalloc_scratch_bytes.restype = C.c_int64
    lib.dsv4_noalloc_scratch_bytes.argtypes = []
    lib.dsv4_attn_last_error.restype = C.c_char_p
    lib.dsv4_attn_last_error.argtypes = []
    lib.dsv4_attn_plan_splits.restype = C.c_int
    lib.dsv4_attn_plan_splits.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int]
    lib.dsv4_attn_workspace_bytes.restype = C.c_int64
    lib.dsv4_attn_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int, P(C.c_int64)]
    # same argument list as the reference binding (bench/bench/candidates/hca_custom_decode.py:60-73)
    lib.hca_decode_fwd.restype = C.c_int
    lib.hca_decode_fwd.argtypes = [C.c_void_p] * 11 + [C.c_float] + [C.c_int] * 6 + [C.c_void_p]
    return lib


LIB = _load()
