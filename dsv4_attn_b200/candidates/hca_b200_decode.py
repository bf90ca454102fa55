"""HCA decode candidate for the reference harness, backed by libdsv4_attn.so.

Drop this file into the reference's `bench/bench/candidates/` folder (or point
`DSV4_HCA_SO` at libdsv4_attn.so and keep using the harness's own
`hca_custom_decode` candidate: the exported `hca_decode_fwd` symbol has the
argument list that module binds, bench/bench/candidates/hca_custom_decode.py:
60-73).  Unlike the harness's own launcher this one accepts any
M_cur + swa_len >= 1, not only multiples of 128.

Interface (bench/bench/candidates/__init__.py:3-6, bench/bench/decode.py:299):
    candidate(inputs: HCADecodeInputs, *, spec: HCADecodeSpec) -> Tensor[B, n_h, c + n_rope]
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

NAME = "hca_b200_decode"
VARIANT = "hca_decode"

_FN = None


def _resolve_so() -> Path:
    for var in ("DSV4_ATTN_SO", "DSV4_HCA_SO"):
        if os.environ.get(var):
            return Path(os.environ[var])
    here = Path(__file__).resolve()
    for parent in here.parents:
        cand = parent / "dsv4_attn_b200" / "libdsv4_attn.so"
        if cand.exists():
            return cand
        cand = parent / "libdsv4_attn.so"
        if cand.exists():
            return cand
    raise RuntimeError("libdsv4_attn.so not found: set DSV4_ATTN_SO or build with `python -m dsv4_attn_b200.build`")


def _load():
    global _FN
    if _FN is not None:
        return _FN
    lib = ctypes.CDLL(str(_resolve_so()))
    fn = lib.hca_decode_fwd
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 11 + [ctypes.c_float] + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    _FN = fn
    return fn


def make_workspace(inputs, *, spec):
    """Output and split workspaces, sized as the harness's own launcher sizes
    them (bench/bench/candidates/hca_custom_decode.py:114-121)."""
    B, n_h, dq = inputs.Q.shape
    dev = inputs.Q.device
    S = max((int(spec.M_cur) + int(spec.swa_len)) // 128, 1)
    O = torch.empty(B, n_h, dq, dtype=torch.bfloat16, device=dev)
    partial_O = torch.empty(S, B, n_h, dq, dtype=torch.float32, device=dev)
    partial_lse = torch.empty(S, B, n_h, dtype=torch.float32, device=dev)
    return O, partial_O, partial_lse


def launch(inputs, *, spec, O, partial_O, partial_lse):
    fn = _load()
    if inputs.Kc_scales is None or inputs.Kswa_scales is None:
        raise ValueError("this candidate reads the FP8 cache: run the harness with --dtype fp8_dequant or fp8")
    u8 = lambda t: (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).contiguous()
    Q = inputs.Q.contiguous()
    Kc, Kc_s, Kc_rope = u8(inputs.Kc), inputs.Kc_scales.contiguous(), inputs.Kc_rope.contiguous()
    Ks, Ks_s, Ks_rope = u8(inputs.Kswa), inputs.Kswa_scales.contiguous(), inputs.Kswa_rope.contiguous()
    sink = inputs.sink_logits.contiguous() if inputs.sink_logits is not None else None
    B, n_h, dq = Q.shape
    c = Kc.shape[-1]
    stream = torch.cuda.current_stream(Q.device).cuda_stream
    rc = fn(Q.data_ptr(), Kc.data_ptr(), Kc_s.data_ptr(), Kc_rope.data_ptr(),
            Ks.data_ptr(), Ks_s.data_ptr(), Ks_rope.data_ptr(),
            sink.data_ptr() if sink is not None else None,
            O.data_ptr(), partial_O.data_ptr(), partial_lse.data_ptr(),
            ctypes.c_float(float(inputs.sm_scale)), B, n_h, c, dq - c,
            int(spec.M_cur), int(spec.swa_len), ctypes.c_void_p(stream))
    if rc != 0:
        raise RuntimeError(f"hca_decode_fwd cudaError={rc}")
    return O


def candidate(inputs, *, spec):
    O, partial_O, partial_lse = make_workspace(inputs, spec=spec)
    return launch(inputs, spec=spec, O=O, partial_O=partial_O, partial_lse=partial_lse)
