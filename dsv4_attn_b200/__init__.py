"""dsv4_attn_b200: decode attention for DeepSeek-V4-style compressed KV caches
on NVIDIA B200 (sm_100a).  CSA sparse decode, HCA dense decode, split-KV merge.

Importing the package loads libdsv4_attn.so and fails if it has not been
built (`python -m dsv4_attn_b200.build`)."""
from . import layout
from ._lib import LIB, library_path
from .api import (Dsv4Error, alloc_workspace, combine, csa_sparse_decode, hca_decode_fwd, hca_dense_decode,
                  new_status, plan_splits)

__all__ = ["LIB", "library_path", "layout", "Dsv4Error", "alloc_workspace", "combine", "csa_sparse_decode",
           "hca_decode_fwd", "hca_dense_decode", "new_status", "plan_splits"]
