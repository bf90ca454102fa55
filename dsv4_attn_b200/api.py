"""Host-side operator surface: torch tensors in, torch tensors out.

Each function follows the pattern of the reference's operator boundary
(csa/interface.h:21-85): check device / dtype / rank / contiguity / shape, fill
a plain parameter struct with raw device pointers, launch on the current
CUDA stream, return tensors the callee allocated (unless the caller passes
them).  The arithmetic is done by libdsv4_attn.so only; nothing here computes
on the host and nothing falls back to PyTorch ops."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from .layout import D_QK, D_LATENT, ENTRY_BYTES, PAGE_ENTRIES

MAX_SPLITS = 64


class Dsv4Error(RuntimeError):
    """A library call returned a non-zero cudaError_t."""


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _cuda_contig(t: torch.Tensor, name: str, dtype, ndim: Optional[int] = None) -> None:
    _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _check(t.is_cuda, f"{name} must be on cuda")
    _check(t.dtype == dtype, f"{name} must be {dtype}, got {t.dtype}")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    if ndim is not None:
        _check(t.dim() == ndim, f"{name} must have {ndim} dims, got {t.dim()}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _rc(rc: int, what: str) -> None:
    if rc != 0:
        raise Dsv4Error(f"{what} failed: cudaError={rc}")


def plan_splits(rows: int, H: int, max_len: int, num_sms: int = 0) -> int:
    """Split count the library's cost model picks (host arithmetic only)."""
    s = _lib.LIB.dsv4_attn_plan_splits(int(rows), int(H), int(max_len), int(num_sms))
    if s < 1:
        raise Dsv4Error(f"dsv4_attn_plan_splits failed: cudaError={-s}")
    return s


def alloc_workspace(rows: int, H: int, num_splits: int, device) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """(partial_o [S, rows, H, 512] f32, partial_lse [S, rows, H] f32) or (None, None)."""
    if num_splits <= 1:
        return None, None
    po = torch.empty(num_splits, rows, H, D_LATENT, dtype=torch.float32, device=device)
    pl = torch.empty(num_splits, rows, H, dtype=torch.float32, device=device)
    return po, pl


def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


class Plan:
    """A split-KV schedule for one batch (see dsv4_attn_plan in include/dsv4_attn.h): the device
    buffer the planner kernel filled, plus the partial-output areas the decode call needs with it.
    A plan depends only on (kind, B, s_q, H) and the length tensors it was made from; it can be
    reused by every layer of a decode step that shares them, and re-made in place with `remake()`
    when the lengths change (same shapes: nothing is allocated)."""

    def __init__(self, kind, B, s_q, H, topk, num_splits, num_sms, lengths, device):
        self.kind, self.B, self.s_q, self.H, self.topk = kind, B, s_q, H, topk
        self.num_splits, self.num_sms = num_splits, num_sms
        po, pl = C.c_int64(0), C.c_int64(0)
        nbytes = _lib.LIB.dsv4_attn_sched_bytes(B * s_q, H, num_splits, num_sms, C.byref(po), C.byref(pl))
        _check(nbytes > 0, "dsv4_attn_sched_bytes rejected the shape")
        self.sched = torch.empty(nbytes // 4, dtype=torch.int32, device=device)
        # one BF16 row of 512 per (slot, head row); held as float32 storage like the split workspace
        self.partial_o = torch.empty(max(po.value // 4, 4), dtype=torch.float32, device=device)
        self.partial_lse = torch.empty(max(pl.value // 4, 4), dtype=torch.float32, device=device)
        self.lengths = lengths
        self.remake()

    def remake(self):
        topk_len, kv_len, win_len = self.lengths
        p = _lib.PlanParams(kind=self.kind, B=self.B, s_q=self.s_q, H=self.H, topk=self.topk, num_splits=self.num_splits,
                            num_sms=self.num_sms, topk_len=_ptr(topk_len), kv_len=_ptr(kv_len), win_len=_ptr(win_len),
                            sched=_ptr(self.sched), sched_bytes=self.sched.numel() * 4)
        rc = _lib.LIB.dsv4_attn_plan(C.byref(p), _stream(self.sched.device))
        if rc != 0:
            raise Dsv4Error(f"dsv4_attn_plan failed: cudaError={rc} {_lib.LIB.dsv4_attn_last_error().decode()}")
        return self

    def info(self):
        """(items, partial slots, capacity exceeded, cost share per block pair): reads the device buffer back."""
        return tuple(self.sched[:4].cpu().tolist())


def plan_csa(B, s_q, H, topk, *, topk_len=None, kv_len=None, num_splits=0, num_sms=0, device="cuda") -> Plan:
    """Schedule for a CSA sparse decode batch.  num_splits = 0: the planner balances the SMs;
    >= 1: exactly that many pieces per (row, 128 heads)."""
    for name, t in (("topk_len", topk_len), ("kv_len", kv_len)):
        if t is not None:
            _cuda_contig(t, name, torch.int32, 2)
            _check(tuple(t.shape) == (B, s_q), f"{name} must be [B, s_q]")
    return Plan(0, B, s_q, H, topk, num_splits, num_sms, (topk_len, kv_len, None), device)


def plan_hca(B, s_q, H, kv_len, win_len, *, num_splits=0, num_sms=0) -> Plan:
    """Schedule for an HCA dense decode batch (lengths int32 [B, s_q] on the device)."""
    _cuda_contig(kv_len, "kv_len", torch.int32, 2)
    _cuda_contig(win_len, "win_len", torch.int32, 2)
    _check(tuple(kv_len.shape) == (B, s_q) and tuple(win_len.shape) == (B, s_q), "kv_len/win_len must be [B, s_q]")
    return Plan(1, B, s_q, H, 0, num_splits, num_sms, (None, kv_len, win_len), kv_len.device)


def check_fp16_operand_range(q: torch.Tensor, kv_pool: torch.Tensor, win_pool: Optional[torch.Tensor] = None) -> None:
    """Host-side check of the preconditions of the FP16 operand route (|q| < 65504, block scales <= 146).
    Reads the tensors back: for callers that cannot vouch for their inputs, not for the hot path."""
    _check(bool(q.abs().max() < 65504), "|q| must stay below 65504")
    for name, pool in (("kv_pool", kv_pool), ("win_pool", win_pool)):
        if pool is not None and pool.numel() > 0:
            sc = pool.reshape(-1, ENTRY_BYTES)[:, 512:528].contiguous().view(torch.float32)
            _check(bool(sc.abs().max() <= 146.0), f"{name}: a block scale exceeds 146 (it would be clamped)")


def _common(q, kv_pool, block_table, attn_sink, out, lse, num_splits, workspace, max_len, need_workspace=True, plan=None):
    _cuda_contig(q, "q", torch.bfloat16, 4)
    B, s_q, H, dq = q.shape
    _check(dq == D_QK, f"q last dim must be {D_QK}")
    _cuda_contig(kv_pool, "kv_pool", torch.uint8, 3)
    _check(kv_pool.shape[1] == PAGE_ENTRIES and kv_pool.shape[2] == ENTRY_BYTES,
           f"kv_pool must be [num_pages, {PAGE_ENTRIES}, {ENTRY_BYTES}]")
    _cuda_contig(block_table, "block_table", torch.int32, 2)
    _check(block_table.shape[0] == B, "block_table must be [B, max_pages]")
    if attn_sink is not None:
        _cuda_contig(attn_sink, "attn_sink", torch.float32, 1)
        _check(attn_sink.shape[0] == H, "attn_sink must be [H]")
    rows = B * s_q
    if plan is not None:
        _check((plan.B, plan.s_q, plan.H) == (B, s_q, H), "plan was made for another batch shape")
        num_splits = 1
        need_workspace = False
    if num_splits is None:
        num_splits = plan_splits(rows, H, max_len)
    _check(1 <= num_splits <= MAX_SPLITS, f"num_splits must be in [1, {MAX_SPLITS}]")
    if out is None:
        out = torch.empty(B, s_q, H, D_LATENT, dtype=torch.bfloat16, device=q.device)
    else:
        _cuda_contig(out, "out", torch.bfloat16, 4)
        _check(tuple(out.shape) == (B, s_q, H, D_LATENT), "out must be [B, s_q, H, 512]")
    if lse is None:
        lse = torch.empty(B, s_q, H, dtype=torch.float32, device=q.device)
    else:
        _cuda_contig(lse, "lse", torch.float32, 3)
        _check(tuple(lse.shape) == (B, s_q, H), "lse must be [B, s_q, H]")
    po = pl = None
    if num_splits > 1 and need_workspace:
        if workspace is None:
            po, pl = alloc_workspace(rows, H, num_splits, q.device)
        else:
            po, pl = workspace
            _cuda_contig(po, "partial_o", torch.float32)
            _cuda_contig(pl, "partial_lse", torch.float32)
            _check(po.numel() >= num_splits * rows * H * D_LATENT and pl.numel() >= num_splits * rows * H,
                   "workspace too small for num_splits")
    if plan is not None:
        po, pl = plan.partial_o, plan.partial_lse
    return B, s_q, H, num_splits, out, lse, po, pl


def csa_sparse_decode(q, kv_pool, block_table, indices, sm_scale, *, kv_len=None, topk_len=None, attn_sink=None,
                      num_splits=None, out=None, lse=None, workspace=None, status=None, impl="mma", plan=None,
                      check_fp16_range=False):
    """CSA sparse decode.  q bf16 [B, s_q, H, 576]; kv_pool uint8 [P, 64, 656];
    block_table int32 [B, max_pages]; indices int32 [B, s_q, topk] (-1 = pad);
    kv_len optional int32 [B, s_q]; topk_len optional int32 [B, s_q] (only the
    first topk_len slots of each list are read).  Returns (out bf16 [B, s_q, H, 512],
    lse f32 [B, s_q, H])."""
    _cuda_contig(indices, "indices", torch.int32, 3)
    topk = indices.shape[-1]
    if impl == "simt":
        num_splits, plan = 1, None
    B, s_q, H, num_splits, out, lse, po, pl = _common(q, kv_pool, block_table, attn_sink, out, lse,
                                                      num_splits, workspace, topk, plan=plan)
    _check(tuple(indices.shape[:2]) == (B, s_q), "indices must be [B, s_q, topk]")
    _check(plan is None or (plan.kind == 0 and plan.topk == topk), "plan was made for another kind of batch")
    if check_fp16_range:
        check_fp16_operand_range(q, kv_pool)
    if kv_len is not None:
        _cuda_contig(kv_len, "kv_len", torch.int32, 2)
        _check(tuple(kv_len.shape) == (B, s_q), "kv_len must be [B, s_q]")
    if topk_len is not None:
        _cuda_contig(topk_len, "topk_len", torch.int32, 2)
        _check(tuple(topk_len.shape) == (B, s_q), "topk_len must be [B, s_q]")
    p = _lib.CsaSparseDecodeParams(
        B=B, s_q=s_q, H=H, topk=topk, max_pages=block_table.shape[1], num_splits=num_splits,
        sm_scale=float(sm_scale), num_pages=kv_pool.shape[0],
        q=_ptr(q), kv_pool=_ptr(kv_pool), block_table=_ptr(block_table), indices=_ptr(indices),
        kv_len=_ptr(kv_len), topk_len=_ptr(topk_len), attn_sink=_ptr(attn_sink), out=_ptr(out), lse=_ptr(lse),
        partial_o=_ptr(po), partial_lse=_ptr(pl), status=_ptr(status), sched=None if plan is None else _ptr(plan.sched))
    fn = _lib.LIB.dsv4_csa_sparse_decode_fwd if impl == "mma" else _lib.LIB.dsv4_csa_sparse_decode_simt
    _rc(fn(C.byref(p), _stream(q.device)), "dsv4_csa_sparse_decode")
    return out, lse


def csa_sparse_decode_noalloc(q, kv_pool, block_table, indices, sm_scale, *, out, lse, num_splits, kv_len=None,
                              topk_len=None, attn_sink=None, status=None):
    """CSA sparse decode through the entry point that allocates nothing.

    For hosts that cannot allocate device memory when they decode (all of HBM
    already given to the KV-cache pool, an allocator they must not touch): the
    split-KV partials go to a fixed 32 MiB array inside the library instead of
    a caller workspace.  `out` and `lse` must be passed in, so that this wrapper
    allocates nothing either.  Raises ValueError when
    num_splits * B * s_q * H * 512 exceeds 8 Mi floats.  Calls share the array:
    do not let two of them overlap on the GPU."""
    _cuda_contig(indices, "indices", torch.int32, 3)
    _check(out is not None and lse is not None, "out and lse must be provided by the caller")
    _check(num_splits is not None, "num_splits must be given")
    B, s_q, H, num_splits, out, lse, _, _ = _common(q, kv_pool, block_table, attn_sink, out, lse, num_splits, None,
                                                    indices.shape[-1], need_workspace=False)
    topk = indices.shape[-1]
    p = _lib.CsaSparseDecodeParams(
        B=B, s_q=s_q, H=H, topk=topk, max_pages=block_table.shape[1], num_splits=num_splits,
        sm_scale=float(sm_scale), num_pages=kv_pool.shape[0],
        q=_ptr(q), kv_pool=_ptr(kv_pool), block_table=_ptr(block_table), indices=_ptr(indices),
        kv_len=_ptr(kv_len), topk_len=_ptr(topk_len), attn_sink=_ptr(attn_sink), out=_ptr(out), lse=_ptr(lse),
        partial_o=None, partial_lse=None, status=_ptr(status))
    rc = _lib.LIB.dsv4_csa_sparse_decode_fwd_noalloc(C.byref(p), _stream(q.device))
    if rc != 0:
        why = _lib.LIB.dsv4_attn_last_error().decode()
        if rc == 1:
            raise ValueError(f"dsv4_csa_sparse_decode_fwd_noalloc rejected the call: {why}")
        raise Dsv4Error(f"dsv4_csa_sparse_decode_fwd_noalloc failed: cudaError={rc} {why}")
    return out, lse


def hca_dense_decode(q, kv_pool, block_table, kv_len, win_pool, win_len, sm_scale, *, attn_sink=None,
                     num_splits=None, out=None, lse=None, workspace=None, status=None, impl="mma",
                     max_len=None, plan=None, check_fp16_range=False):
    """HCA dense decode.  kv_len / win_len int32 [B, s_q]; win_pool uint8
    [B, W, 656].  `max_len` (longest kv_len + win_len) only steers the split
    planner; when omitted the block-table capacity is used so that no device
    read-back is needed."""
    _cuda_contig(kv_len, "kv_len", torch.int32, 2)
    _cuda_contig(win_len, "win_len", torch.int32, 2)
    _cuda_contig(win_pool, "win_pool", torch.uint8, 3)
    _check(win_pool.shape[2] == ENTRY_BYTES, "win_pool must be [B, W, 656]")
    W = win_pool.shape[1]
    if max_len is None:
        max_len = block_table.shape[1] * PAGE_ENTRIES + W
    if impl == "simt":
        num_splits, plan = 1, None
    B, s_q, H, num_splits, out, lse, po, pl = _common(q, kv_pool, block_table, attn_sink, out, lse,
                                                      num_splits, workspace, max_len, plan=plan)
    _check(plan is None or plan.kind == 1, "plan was made for another kind of batch")
    if check_fp16_range:
        check_fp16_operand_range(q, kv_pool, win_pool)
    _check(tuple(kv_len.shape) == (B, s_q) and tuple(win_len.shape) == (B, s_q), "kv_len/win_len must be [B, s_q]")
    _check(win_pool.shape[0] == B, "win_pool must be [B, W, 656]")
    p = _lib.HcaDenseDecodeParams(
        B=B, s_q=s_q, H=H, max_pages=block_table.shape[1], win_cap=W, num_splits=num_splits,
        sm_scale=float(sm_scale), num_pages=kv_pool.shape[0],
        q=_ptr(q), kv_pool=_ptr(kv_pool), block_table=_ptr(block_table), kv_len=_ptr(kv_len),
        win_pool=_ptr(win_pool), win_len=_ptr(win_len), attn_sink=_ptr(attn_sink),
        out=_ptr(out), lse=_ptr(lse), partial_o=_ptr(po), partial_lse=_ptr(pl), status=_ptr(status),
        sched=None if plan is None else _ptr(plan.sched))
    fn = _lib.LIB.dsv4_hca_dense_decode_fwd if impl == "mma" else _lib.LIB.dsv4_hca_dense_decode_simt
    _rc(fn(C.byref(p), _stream(q.device)), "dsv4_hca_dense_decode")
    return out, lse


def combine(partial_o, partial_lse, *, attn_sink=None, out=None, lse=None):
    """Merge split partials: partial_o f32 [S, N, H, 512], partial_lse f32
    [S, N, H] (log2).  Returns (out bf16 [N, H, 512], lse f32 [N, H])."""
    _cuda_contig(partial_o, "partial_o", torch.float32, 4)
    _cuda_contig(partial_lse, "partial_lse", torch.float32, 3)
    S, N, H, D = partial_o.shape
    _check(D == D_LATENT, "partial_o last dim must be 512")
    _check(tuple(partial_lse.shape) == (S, N, H), "partial_lse must be [S, N, H]")
    if attn_sink is not None:
        _cuda_contig(attn_sink, "attn_sink", torch.float32, 1)
    if out is None:
        out = torch.empty(N, H, D, dtype=torch.bfloat16, device=partial_o.device)
    if lse is None:
        lse = torch.empty(N, H, dtype=torch.float32, device=partial_o.device)
    p = _lib.CombineParams(
        N=N, H=H, D=D, num_splits=S, partial_o=_ptr(partial_o), partial_lse=_ptr(partial_lse),
        out=_ptr(out), lse=_ptr(lse), attn_sink=_ptr(attn_sink),
        stride_po_split=N * H * D, stride_po_n=H * D, stride_po_h=D,
        stride_pl_split=N * H, stride_pl_n=H, stride_out_n=H * D, stride_out_h=D, stride_lse_n=H)
    _rc(_lib.LIB.dsv4_attn_combine(C.byref(p), _stream(partial_o.device)), "dsv4_attn_combine")
    return out, lse


def hca_decode_fwd(Q, Kc, Kc_s, Kc_rope, Kswa, Kswa_s, Kswa_rope, sink_logits, sm_scale, *, M_cur, swa_len,
                   O=None, partial_O=None, partial_lse=None):
    """The reference's entry point on its own cache layout (448 e4m3 + 7 UE8M0
    + 64 bf16 per entry), same arguments as the reference's ctypes launcher
    (bench/bench/candidates/hca_custom_decode.py:124-158)."""
    _cuda_contig(Q, "Q", torch.bfloat16, 3)
    B, n_h, dq = Q.shape
    c = Kc.shape[-1]
    n_rope = dq - c
    if O is None:
        O = torch.empty(B, n_h, dq, dtype=torch.bfloat16, device=Q.device)
    S = (M_cur + swa_len) // 128
    if partial_O is None and S > 1:
        partial_O = torch.empty(S, B, n_h, dq, dtype=torch.float32, device=Q.device)
        partial_lse = torch.empty(S, B, n_h, dtype=torch.float32, device=Q.device)
    u8 = lambda t: t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t
    rc = _lib.LIB.hca_decode_fwd(
        _ptr(Q), _ptr(u8(Kc)), _ptr(Kc_s), _ptr(Kc_rope), _ptr(u8(Kswa)), _ptr(Kswa_s), _ptr(Kswa_rope),
        _ptr(sink_logits), _ptr(O), _ptr(partial_O), _ptr(partial_lse),
        C.c_float(float(sm_scale)), B, n_h, c, n_rope, int(M_cur), int(swa_len), _stream(Q.device))
    _rc(rc, "hca_decode_fwd")
    return O


def csa_compress_reduce_fwd(C_a, C_b, Z_a, Z_b, B_a, B_b, m, *, out=None):
    """CSA compressor, second pass.  Same arguments, checks and result as the
    reference's csa_compress_reduce_fwd (csa/interface.h:21-85, bound in
    csa/pybind.cpp:5-17): four BF16 streams [B, n, c_out], two BF16 biases
    [m, c_out], returns BF16 [B, n/m, c_out] allocated here."""
    for name, t in (("C_a", C_a), ("C_b", C_b), ("Z_a", Z_a), ("Z_b", Z_b)):
        _check(t.is_cuda, "all inputs must be on cuda")
        _check(t.dtype == torch.bfloat16, f"{name} must be bf16")
        _check(t.is_contiguous(), "input streams must be contiguous")
    _check(B_a.dtype == torch.bfloat16 and B_b.dtype == torch.bfloat16, "biases must be bf16")
    _check(B_a.is_cuda and B_b.is_cuda and B_a.is_contiguous() and B_b.is_contiguous(), "biases must be contiguous cuda tensors")
    _check(C_a.dim() == 3 and C_a.shape == C_b.shape == Z_a.shape == Z_b.shape,
           "C_a/C_b/Z_a/Z_b must all be [B, n, c_out] and equal-shaped")
    _check(B_a.dim() == 2 and B_a.shape[0] == m and B_b.dim() == 2 and B_b.shape[0] == m, "B_a/B_b must be [m, c_out]")
    B, n, c_out = C_a.shape
    _check(B_a.shape[1] == c_out and B_b.shape[1] == c_out, "B_a/B_b last dim must match c_out")
    _check(n % m == 0, "n must be divisible by m")
    _check(m == 4, f"[dsv4-csa] unsupported m={m} (only m=4 instantiated)")
    if out is None:
        out = torch.empty(B, n // m, c_out, dtype=torch.bfloat16, device=C_a.device)
    p = _lib.CsaCompressReduceParams(
        B=B, n=n, c_out=c_out, m=m, C_a=_ptr(C_a), C_b=_ptr(C_b), Z_a=_ptr(Z_a), Z_b=_ptr(Z_b),
        B_a=_ptr(B_a), B_b=_ptr(B_b), out=_ptr(out), stride_C_b=n * c_out, stride_C_n=c_out,
        stride_out_b=(n // m) * c_out, stride_out_blk=c_out)
    _rc(_lib.LIB.dsv4_csa_compress_reduce_fwd(C.byref(p), _stream(C_a.device)), "dsv4_csa_compress_reduce_fwd")
    return out


def _cache_dest(kv_pool, block_table, insert_pos, status, B):
    _cuda_contig(kv_pool, "kv_pool", torch.uint8, 3)
    _check(kv_pool.shape[1] == PAGE_ENTRIES and kv_pool.shape[2] == ENTRY_BYTES, f"kv_pool must be [pages, {PAGE_ENTRIES}, {ENTRY_BYTES}]")
    _cuda_contig(block_table, "block_table", torch.int32, 2)
    _cuda_contig(insert_pos, "insert_pos", torch.int32, 1)
    _check(block_table.shape[0] == B and insert_pos.shape[0] == B, "block_table / insert_pos must have one row per request")
    if status is not None:
        _cuda_contig(status, "status", torch.int32, 1)
        _check(status.numel() >= 4, "status must hold 4 int32")
    return _lib.CacheDest(kv_pool=_ptr(kv_pool), block_table=_ptr(block_table), insert_pos=_ptr(insert_pos),
                          max_pages=block_table.shape[1], num_pages=kv_pool.shape[0], status=_ptr(status))


def hca_compress_fwd(C_, Z, bias, m, *, out=None, kv_pool=None, block_table=None, insert_pos=None, status=None,
                     want_out=True):
    """HCA compressor: BF16 streams C, Z [B, n, c] and bias [m, c] -> BF16 [B, n/m, c]
    (the reduce of the reference's compressor_simple, bench/bench/reference.py:117-122).
    With kv_pool / block_table / insert_pos (c == 576) the rows are also quantised and
    written into the paged cache as entries insert_pos[b] + i; `want_out=False` skips the
    dense output then."""
    for name, t in (("C", C_), ("Z", Z)):
        _cuda_contig(t, name, torch.bfloat16, 3)
    _check(C_.shape == Z.shape, "C and Z must be equal-shaped [B, n, c]")
    _cuda_contig(bias, "bias", torch.bfloat16, 2)
    B, n, c = C_.shape
    _check(bias.shape[0] == m and bias.shape[1] == c, "bias must be [m, c]")
    _check(m >= 1 and n % m == 0, "n must be divisible by m")
    _check(c % 8 == 0, "c must be a multiple of 8")
    dst = None
    if kv_pool is not None:
        _check(c == D_QK, f"the cache insert needs c == {D_QK}")
        dst = _cache_dest(kv_pool, block_table, insert_pos, status, B)
    _check(want_out or dst is not None, "nothing to produce")
    if want_out and out is None:
        out = torch.empty(B, n // m, c, dtype=torch.bfloat16, device=C_.device)
    if out is not None:
        _cuda_contig(out, "out", torch.bfloat16, 3)
        _check(tuple(out.shape) == (B, n // m, c), "out must be [B, n/m, c]")
    p = _lib.HcaCompressParams(B=B, n=n, c=c, m=m, C=_ptr(C_), Z=_ptr(Z), bias=_ptr(bias), stride_b=n * c, stride_n=c,
                               out=_ptr(out), dst=C.pointer(dst) if dst is not None else None)
    _rc(_lib.LIB.dsv4_hca_compress_fwd(C.byref(p), _stream(C_.device)), "dsv4_hca_compress_fwd")
    return out


def kv_quantize_insert(rows, kv_pool, block_table, insert_pos, *, n_rows=None, status=None) -> None:
    """Quantise BF16 rows [B, T, 576] into 656-byte cache entries and write them at logical
    positions insert_pos[b] + t of request b (in place, into kv_pool)."""
    _cuda_contig(rows, "rows", torch.bfloat16, 3)
    B, T, c = rows.shape
    _check(c == D_QK, f"rows must be [B, T, {D_QK}]")
    dst = _cache_dest(kv_pool, block_table, insert_pos, status, B)
    if n_rows is not None:
        _cuda_contig(n_rows, "n_rows", torch.int32, 1)
        _check(n_rows.shape[0] == B, "n_rows must be [B]")
    p = _lib.KvQuantizeInsertParams(B=B, T=T, rows=_ptr(rows), stride_b=T * c, stride_t=c, n_rows=_ptr(n_rows),
                                    dst=C.pointer(dst))
    _rc(_lib.LIB.dsv4_kv_quantize_insert(C.byref(p), _stream(rows.device)), "dsv4_kv_quantize_insert")


REF_TOKEN_BYTES = 576      # 448 e4m3 latent + 64 BF16 RoPE values
REF_PAGE_TOKEN_BYTES = 584 # + 7 UE8M0 scale bytes and 1 pad byte in the page's scale area


def hca_packed_decode(q, kv_pages, block_table, m_cur, swa_pages, swa_block_table, swa_len, sm_scale, *,
                      page_size=64, attn_sink=None, num_splits=None, out=None, lse=None, workspace=None, status=None):
    """HCA decode over packed cache pages in the reference's byte format (see
    Dsv4HcaPackedDecodeParams in include/dsv4_attn.h), per-request lengths m_cur / swa_len
    int32 [B].  q bf16 [B, H, 512]; pools uint8 [pages, page_size*584].  Returns
    (out bf16 [B, H, 512], lse f32 [B, H])."""
    _cuda_contig(q, "q", torch.bfloat16, 3)
    B, H, dq = q.shape
    _check(dq == 512, "q must be [B, H, 512]")
    _check(page_size in (16, 32, 64), "page_size must be 16, 32 or 64")
    for name, pool, table in (("kv_pages", kv_pages, block_table), ("swa_pages", swa_pages, swa_block_table)):
        if pool is None:
            continue
        _cuda_contig(pool, name, torch.uint8, 2)
        _check(pool.shape[1] == page_size * REF_PAGE_TOKEN_BYTES, f"{name} must be [pages, page_size*{REF_PAGE_TOKEN_BYTES}]")
        _cuda_contig(table, name + " block table", torch.int32, 2)
        _check(table.shape[0] == B, "block tables must have one row per request")
    _check(kv_pages is not None or swa_pages is not None, "at least one pool is needed")
    _cuda_contig(m_cur, "m_cur", torch.int32, 1)
    _cuda_contig(swa_len, "swa_len", torch.int32, 1)
    _check(m_cur.shape[0] == B and swa_len.shape[0] == B, "m_cur / swa_len must be [B]")
    if attn_sink is not None:
        _cuda_contig(attn_sink, "attn_sink", torch.float32, 1)
        _check(attn_sink.shape[0] == H, "attn_sink must be [H]")
    cap = (block_table.shape[1] if kv_pages is not None else 0) * page_size + \
          (swa_block_table.shape[1] if swa_pages is not None else 0) * page_size
    if num_splits is None:
        num_splits = plan_splits(B, H, cap)
    _check(1 <= num_splits <= MAX_SPLITS, "num_splits out of range")
    if out is None:
        out = torch.empty(B, H, 512, dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty(B, H, dtype=torch.float32, device=q.device)
    po, pl = workspace if workspace is not None else alloc_workspace(B, H, num_splits, q.device)
    p = _lib.HcaPackedDecodeParams(
        B=B, H=H, page_size=page_size, max_pages=block_table.shape[1] if kv_pages is not None else 0,
        swa_max_pages=swa_block_table.shape[1] if swa_pages is not None else 0, num_splits=num_splits,
        sm_scale=float(sm_scale), num_pages=kv_pages.shape[0] if kv_pages is not None else 0,
        swa_num_pages=swa_pages.shape[0] if swa_pages is not None else 0,
        q=_ptr(q), kv_pages=_ptr(kv_pages), block_table=_ptr(block_table) if kv_pages is not None else None, m_cur=_ptr(m_cur),
        swa_pages=_ptr(swa_pages), swa_block_table=_ptr(swa_block_table) if swa_pages is not None else None,
        swa_len=_ptr(swa_len), attn_sink=_ptr(attn_sink), out=_ptr(out), lse=_ptr(lse),
        partial_o=_ptr(po), partial_lse=_ptr(pl), status=_ptr(status))
    _rc(_lib.LIB.dsv4_hca_packed_decode_fwd(C.byref(p), _stream(q.device)), "dsv4_hca_packed_decode_fwd")
    return out, lse


def rope_norm(x, positions, *, norm_weight=None, eps=1e-6, n_rope=64, theta=10000.0, inverse=False, out=None):
    """Partial RoPE on the last n_rope dims of x [rows, vecs, c] (bf16) by positions [rows]
    (int32), then an RMS norm over the whole vector when norm_weight [c] is given (the
    reference's apply_rope followed by rms_norm, bench/bench/reference.py:35-70, 281-287).
    `inverse=True` rotates by -position (the inverse RoPE on the attention output,
    reference.py:308-309).  `out` may be x itself."""
    _cuda_contig(x, "x", torch.bfloat16, 3)
    rows, vecs, c = x.shape
    _cuda_contig(positions, "positions", torch.int32, 1)
    _check(positions.shape[0] == rows, "positions must be [rows]")
    _check(n_rope == 64 and c >= 64 and (c - 64) % 8 == 0 and c - 64 <= 512, "unsupported vector width")
    if norm_weight is not None:
        _cuda_contig(norm_weight, "norm_weight", torch.bfloat16, 1)
        _check(norm_weight.shape[0] == c, "norm_weight must be [c]")
    if out is None:
        out = torch.empty_like(x)
    _cuda_contig(out, "out", torch.bfloat16, 3)
    _check(out.shape == x.shape, "out must have the shape of x")
    p = _lib.RopeNormParams(n_rows=rows, vecs_per_row=vecs, c=c, n_rope=n_rope, inverse=1 if inverse else 0, eps=float(eps),
                            theta=float(theta), x=_ptr(x), out=_ptr(out), positions=_ptr(positions), norm_weight=_ptr(norm_weight))
    _rc(_lib.LIB.dsv4_rope_norm_fwd(C.byref(p), _stream(x.device)), "dsv4_rope_norm_fwd")
    return out


INDEXER_HEADS = 64
INDEXER_DIM = 128
INDEXER_PAGE_BYTES = 64 * 128 + 64 * 4


def indexer_topk(q_fp8, q_weight, key_pages, block_table, n_vis, k, *, scores=None, out=None, status=None):
    """CSA indexer for decode: top-k visible entries per query token (see
    Dsv4IndexerTopkParams).  q_fp8 uint8 [B, s_q, 64, 128] (e4m3), q_weight f32 [B, s_q, 64],
    key_pages uint8 [pages, 8448], block_table int32 [B, max_pages], n_vis int32 [B, s_q].
    Returns (indices int32 [B, s_q, k], scores f32 [B*s_q, stride])."""
    _cuda_contig(q_fp8, "q_fp8", torch.uint8, 4)
    B, s_q, nh, dim = q_fp8.shape
    _check(nh == INDEXER_HEADS and dim == INDEXER_DIM, "q_fp8 must be [B, s_q, 64, 128]")
    _check(s_q in (1, 2), "s_q must be 1 or 2")
    _cuda_contig(q_weight, "q_weight", torch.float32, 3)
    _check(tuple(q_weight.shape) == (B, s_q, nh), "q_weight must be [B, s_q, 64]")
    _cuda_contig(key_pages, "key_pages", torch.uint8, 2)
    _check(key_pages.shape[1] == INDEXER_PAGE_BYTES, f"key_pages must be [pages, {INDEXER_PAGE_BYTES}]")
    _cuda_contig(block_table, "block_table", torch.int32, 2)
    _check(block_table.shape[0] == B, "block_table must have one row per request")
    _cuda_contig(n_vis, "n_vis", torch.int32, 2)
    _check(tuple(n_vis.shape) == (B, s_q), "n_vis must be [B, s_q]")
    _check(k >= 1, "k must be positive")
    stride = block_table.shape[1] * 64
    if scores is None:
        scores = torch.empty(B * s_q, stride, dtype=torch.float32, device=q_fp8.device)
    _cuda_contig(scores, "scores", torch.float32, 2)
    _check(scores.shape[0] == B * s_q and scores.shape[1] >= stride, "scores must be [B*s_q, >= max_pages*64]")
    if out is None:
        out = torch.empty(B, s_q, k, dtype=torch.int32, device=q_fp8.device)
    _cuda_contig(out, "out", torch.int32, 3)
    _check(tuple(out.shape) == (B, s_q, k), "out must be [B, s_q, k]")
    p = _lib.IndexerTopkParams(B=B, s_q=s_q, max_pages=block_table.shape[1], k=k, num_pages=key_pages.shape[0],
                               score_stride=scores.shape[1], q_fp8=_ptr(q_fp8), q_weight=_ptr(q_weight), key_pages=_ptr(key_pages),
                               block_table=_ptr(block_table), n_vis=_ptr(n_vis), scores=_ptr(scores), out_indices=_ptr(out),
                               status=_ptr(status))
    _rc(_lib.LIB.dsv4_indexer_topk_fwd(C.byref(p), _stream(q_fp8.device)), "dsv4_indexer_topk_fwd")
    return out, scores
