"""Generate the golden fixtures in this directory from the reference project.

Run where the reference checkout is available:

    python tests/golden/gen_golden.py --reference /path/to/reference

It imports the reference's PyTorch decode path (`bench.reference`), feeds it
the seeded inputs built by `oracle/dsv4_oracle.py`, and stores the reference's
OUTPUTS (plus a hash of the inputs) as small `.npz` files.  The tests rebuild
the inputs from the same seeds, so the fixtures stay small and the reference
checkout is not needed to run the tests.

What each fixture pins:
  csa_cfg0 / csa_ragged / hca_small: gather (reference.py:576-580, torch.gather
      on the un-paged, exactly dequantised pool) followed by
      hca_decode_forward(dtype="fp32") (reference.py:471-546), first 512 output
      columns.
  ref_layout: hca_decode_forward(dtype="fp8_dequant") and dtype="fp8" on the
      reference's own 448+7+64 cache layout.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))

from oracle import dsv4_oracle as orc  # noqa: E402


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def bf16_bits(t):
    import torch
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def ref_attend(ref, q, rows, sm_scale, sink):
    """q [H,576] f32, rows [n,576] f32 -> reference output bits [H,512]."""
    import torch
    H = q.shape[0]
    Q = torch.from_numpy(q).to(torch.bfloat16).unsqueeze(0)
    kv = torch.from_numpy(rows).unsqueeze(0)
    empty = torch.zeros(1, 0, orc.D_LATENT)
    empty_r = torch.zeros(1, 0, orc.D_ROPE)
    s = torch.full((H,), float("-inf")) if sink is None else torch.from_numpy(sink)
    inp = ref.HCADecodeInputs(
        Q=Q, Kc=kv[..., :orc.D_LATENT].contiguous(), Kc_rope=kv[..., orc.D_LATENT:].contiguous(),
        Kc_scales=None, Kswa=empty, Kswa_rope=empty_r, Kswa_scales=None,
        sink_logits=s, sm_scale=sm_scale)
    o = ref.hca_decode_forward(inp, dtype="fp32")
    return bf16_bits(o[0, :, :orc.D_LATENT])


def gen_csa(ref, name, **kw):
    import torch
    case = orc.make_csa_case(**kw)
    B, s_q, H, _ = case.q.shape
    out = np.zeros((B, s_q, H, orc.D_LATENT), np.uint16)
    for b in range(B):
        # un-page this request's cache, as the reference has no paging
        n_pages = case.block_table.shape[1]
        flat = case.pool[case.block_table[b]].reshape(n_pages * orc.PAGE_ENTRIES, orc.ENTRY_BYTES)
        deq = torch.from_numpy(orc.unpack_entries(flat))
        for j in range(s_q):
            idx = case.indices[b, j]
            ok = (idx >= 0) & (idx < case.kv_len[b, j])
            sel = torch.from_numpy(idx[ok].astype(np.int64))
            # the reference's gather step (reference.py:576-580)
            rows = torch.gather(deq, 0, sel.unsqueeze(-1).expand(-1, deq.shape[-1]))
            out[b, j] = ref_attend(ref, case.q[b, j], rows.numpy(), case.sm_scale, None)
    np.savez_compressed(HERE / f"{name}.npz", out=out,
                        inputs_sha=sha(case.q, case.pool, case.block_table, case.indices),
                        kwargs=repr(kw))
    print(name, out.shape)


def gen_hca(ref, name, **kw):
    case = orc.make_hca_case(**kw)
    B, s_q, H, _ = case.q.shape
    out = np.zeros((B, s_q, H, orc.D_LATENT), np.uint16)
    for b in range(B):
        for j in range(s_q):
            n, w = int(case.kv_len[b, j]), int(case.win_len[b, j])
            rows = orc.gather_rows(case.pool, case.block_table[b], np.arange(n))
            rows = np.concatenate([rows, case.win[b, :w]], axis=0)
            out[b, j] = ref_attend(ref, case.q[b, j], orc.unpack_entries(rows), case.sm_scale, case.sink)
    np.savez_compressed(HERE / f"{name}.npz", out=out,
                        inputs_sha=sha(case.q, case.pool, case.block_table, case.win),
                        kwargs=repr(kw))
    print(name, out.shape)


def gen_ref_layout(ref, name, **kw):
    import torch
    c = orc.make_ref_layout_case(**kw)
    t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)) if dt is None else torch.from_numpy(np.ascontiguousarray(a)).to(dt)
    inp = ref.HCADecodeInputs(
        Q=t(c.Q, torch.bfloat16),
        Kc=t(c.Kc).view(torch.float8_e4m3fn), Kc_rope=t(c.Kc_rope, torch.bfloat16), Kc_scales=t(c.Kc_s),
        Kswa=t(c.Kswa).view(torch.float8_e4m3fn), Kswa_rope=t(c.Kswa_rope, torch.bfloat16), Kswa_scales=t(c.Kswa_s),
        sink_logits=t(c.sink), sm_scale=c.sm_scale)
    o_deq = bf16_bits(ref.hca_decode_forward(inp, dtype="fp8_dequant"))
    o_fp8 = bf16_bits(ref.hca_decode_forward(inp, dtype="fp8"))
    np.savez_compressed(HERE / f"{name}.npz", out_fp8_dequant=o_deq, out_fp8=o_fp8,
                        inputs_sha=sha(c.Q, c.Kc, c.Kc_s, c.Kc_rope, c.Kswa, c.Kswa_s, c.Kswa_rope, c.sink),
                        kwargs=repr(kw))
    print(name, o_deq.shape)


def gen_compress(ref, name, **kw):
    """compressor_overlap (reference.py:125-155) fed with selection matrices as
    weights, so that its projections reproduce the four given streams exactly
    and only its gated reduce (Eqs 11-12) is exercised."""
    import torch
    c = orc.make_compress_case(**kw)
    B, n, co = c.C_a.shape
    H = torch.from_numpy(np.concatenate([c.C_a, c.C_b, c.Z_a, c.Z_b], axis=-1))       # [B, n, 4*co]
    sel = lambda k: torch.cat([torch.eye(co) if i == k else torch.zeros(co, co) for i in range(4)], dim=0)
    w = ref.CompressorWeightsOverlap(W_a_KV=sel(0), W_b_KV=sel(1), W_a_Z=sel(2), W_b_Z=sel(3),
                                     B_a=torch.from_numpy(c.B_a), B_b=torch.from_numpy(c.B_b))
    out = ref.compressor_overlap(H, w, c.m)
    np.savez_compressed(HERE / f"{name}.npz", out=bf16_bits(out),
                        inputs_sha=sha(c.C_a, c.C_b, c.Z_a, c.Z_b, c.B_a, c.B_b), kwargs=repr(kw))
    print(name, tuple(out.shape))


def gen_hca_compress(ref, name, **kw):
    """compressor_simple (reference.py:108-122) fed with selection matrices as
    weights, so that its projections reproduce the two given streams exactly and
    only its softmax-weighted reduce is exercised.  Stored as float32."""
    import torch
    c = orc.make_hca_compress_case(**kw)
    B, n, co = c.C.shape
    H = torch.from_numpy(np.concatenate([c.C, c.Z], axis=-1))                           # [B, n, 2*co]
    sel = lambda k: torch.cat([torch.eye(co) if i == k else torch.zeros(co, co) for i in range(2)], dim=0)
    w = ref.CompressorWeightsSimple(W_a_KV=sel(0), W_a_Z=sel(1), B_a=torch.from_numpy(c.bias))
    out = ref.compressor_simple(H, w, c.m)
    np.savez_compressed(HERE / f"{name}.npz", out=out.numpy().astype(np.float32),
                        inputs_sha=sha(c.C, c.Z, c.bias), kwargs=repr(kw))
    print(name, tuple(out.shape))


def make_rope_norm_inputs(seed, rows, vecs, c, max_pos):
    rng = np.random.default_rng(seed)
    x = orc.bf16_round(rng.standard_normal((rows, vecs, c), dtype=np.float32))
    pos = rng.integers(0, max_pos, size=rows).astype(np.int32)
    w = orc.bf16_round((1.0 + 0.1 * rng.standard_normal(c)).astype(np.float32))
    return x, pos, w


def gen_rope_norm(ref, name, **kw):
    """apply_rope (+ rms_norm) of the reference on BF16-representable float32 inputs:
    `q` = RoPE by +pos then norm (reference.py:281-287), `o` = RoPE by -pos, no norm
    (reference.py:308-309).  Stored as float32."""
    import torch
    x, pos, w = make_rope_norm_inputs(**kw)
    xt = torch.from_numpy(x)
    p = torch.from_numpy(pos).unsqueeze(1).expand(-1, x.shape[1])
    q = ref.rms_norm(ref.apply_rope(xt, p, 64), torch.from_numpy(w), 1e-6)
    o = ref.apply_rope(xt, -p, 64)
    np.savez_compressed(HERE / f"{name}.npz", q=q.numpy().astype(np.float32), o=o.numpy().astype(np.float32),
                        inputs_sha=sha(x, pos, w), kwargs=repr(kw))
    print(name, tuple(q.shape))


def gen_indexer(ref, name, **kw):
    """lightning_indexer_topk (reference.py:169-205) with identity projections, so that its
    q_I / w_I are the given ones: n = nb * m tokens, only the two query tokens of the case
    carry a query; their visible blocks are floor(t / m).  Stores the selected block ids."""
    import torch
    m, top_k = kw["m"], kw["top_k"]
    kwc = {k: v for k, v in kw.items() if k not in ("m", "top_k", "tokens")}
    c = orc.make_indexer_case(**kwc)
    B, s_q = c.n_vis.shape
    nb = c.K.shape[1]
    n = nb * m
    k8, ksc = orc.quantize_indexer_keys(c.K)
    K_deq = (orc.e4m3_to_f32(k8) * ksc[..., None]).astype(np.float32)
    d = orc.IDX_HEADS * orc.IDX_DIM
    c_Q = np.zeros((B, n, d), np.float32)
    Hw = np.zeros((B, n, orc.IDX_HEADS), np.float32)
    toks = kw["tokens"]
    for j, t in enumerate(toks):
        c_Q[:, t] = (orc.e4m3_to_f32(c.q_fp8[:, j]) * c.q_scale[:, j, :, None]).reshape(B, d)
        Hw[:, t] = c.w[:, j]
    w = ref.IndexerWeights(W_IUQ=torch.eye(d), W_w=torch.eye(orc.IDX_HEADS), n_heads=orc.IDX_HEADS, head_dim=orc.IDX_DIM)
    sel = ref.lightning_indexer_topk(torch.from_numpy(Hw), torch.from_numpy(c_Q), torch.from_numpy(K_deq), w, m, top_k)
    sel = sel[:, toks].numpy().astype(np.int32)                       # [B, s_q, top_k], best first
    np.savez_compressed(HERE / f"{name}.npz", sel=sel, n_vis=np.array([[t // m for t in toks]] * B, np.int32),
                        inputs_sha=sha(c.q_fp8, c.q_scale, c.w, c.K), kwargs=repr(kw))
    print(name, sel.shape)


# The cases; tests/test_oracle.py rebuilds the inputs from the same kwargs.
CSA_CASES = {
    "csa_cfg0": dict(seed=0, B=2, s_q=1, H=16, n_entries=1024, topk=256),
    "csa_ragged": dict(seed=1, B=3, s_q=2, H=16, n_entries=[100, 300, 37], topk=128, ragged=True),
}
HCA_CASES = {
    "hca_small": dict(seed=2, B=2, s_q=1, H=16, kv_len=[150, 70], win_len=[128, 5], with_sink=True),
    "hca_nosink": dict(seed=3, B=2, s_q=2, H=8, kv_len=[64, 1], win_len=[2, 128]),
}
COMPRESS_CASES = {
    "csa_compress": dict(seed=6, B=2, n=64, c_out=128),
    "csa_compress_odd": dict(seed=7, B=1, n=12, c_out=20),
}
HCA_COMPRESS_CASES = {
    "hca_compress": dict(seed=8, B=2, n=256, c=576),
    "hca_compress_m16": dict(seed=9, B=1, n=48, c=40, m=16),
}
ROPE_NORM_CASES = {
    "rope_norm_q576": dict(seed=12, rows=6, vecs=16, c=576, max_pos=4096),
    "rope_norm_o512": dict(seed=13, rows=5, vecs=8, c=512, max_pos=100000),
}
INDEXER_CASES = {
    "indexer_topk": dict(seed=14, B=1, s_q=2, n=300, m=4, top_k=64, tokens=[1195, 1199]),
}
REF_CASES = {
    "ref_layout": dict(seed=4, B=1, H=128, M_cur=192, swa_len=64),
    "ref_layout_ragged": dict(seed=5, B=2, H=32, M_cur=77, swa_len=19),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DSV4_REFERENCE"))
    args = ap.parse_args()
    if not args.reference or not (Path(args.reference) / "bench" / "bench" / "reference.py").exists():
        print("give --reference /path/to/the/reference/checkout or set DSV4_REFERENCE", file=sys.stderr)
        return 2
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(Path(args.reference) / "bench"))
    from bench import reference as ref  # the reference's own module

    for name, kw in CSA_CASES.items():
        gen_csa(ref, name, **kw)
    for name, kw in HCA_CASES.items():
        gen_hca(ref, name, **kw)
    for name, kw in REF_CASES.items():
        gen_ref_layout(ref, name, **kw)
    for name, kw in COMPRESS_CASES.items():
        gen_compress(ref, name, **kw)
    for name, kw in HCA_COMPRESS_CASES.items():
        gen_hca_compress(ref, name, **kw)
    for name, kw in ROPE_NORM_CASES.items():
        gen_rope_norm(ref, name, **kw)
    for name, kw in INDEXER_CASES.items():
        gen_indexer(ref, name, **kw)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
