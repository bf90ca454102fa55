"""dsv4_attn_b200: decode attention for DeepSeek-V4-style compressed KV caches
on NVIDIA B200 (sm_100a).  CSA sparse decode, HCA dense decode, split-KV merge.

The operators live in libdsv4_attn.so (built by `python -m dsv4_attn_b200.build`).
The shared object is loaded on first use of any operator or of `LIB`; if it is
missing or stale that access raises - there is no CPU or PyTorch fallback.
Importing the bare package stays possible so that the build module can run."""
from __future__ import annotations

import importlib

_API = ("Dsv4Error", "alloc_workspace", "combine", "csa_sparse_decode", "csa_sparse_decode_noalloc", "csa_compress_reduce_fwd", "hca_compress_fwd", "kv_quantize_insert", "hca_packed_decode", "rope_norm", "indexer_topk", "hca_decode_fwd", "hca_dense_decode",
        "new_status", "plan_splits", "plan_csa", "plan_hca", "Plan", "check_fp16_operand_range")
__all__ = ["LIB", "library_path", "layout", "synth", *_API]


def __getattr__(name):
    if name in _API:
        return getattr(importlib.import_module(".api", __name__), name)
    if name in ("LIB", "library_path"):
        return getattr(importlib.import_module("._lib", __name__), name)
    if name in ("layout", "synth", "api", "build"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
