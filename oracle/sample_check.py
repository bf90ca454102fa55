"""TEST INFRASTRUCTURE ONLY.  Checks rows of a decode result that lives on the device against the
CPU oracle: the cache entries of the sampled rows are gathered on the device (a plain index
operation), brought to the host and run through dsv4_oracle.attend.  Used by the GPU tests at sizes
where the whole batch is too much for the numpy oracle, and by bench.py after its timed regions."""
from __future__ import annotations

import numpy as np
import torch

from . import dsv4_oracle as orc


def _compare(got_out, got_lse, want_out_bits, want_lse):
    want = orc.bf16_bits_to_f32(want_out_bits)
    err = np.abs(got_out - want)
    inf = np.isneginf(want_lse)
    ok_inf = bool(np.array_equal(np.isneginf(got_lse), inf))
    fin = ~inf
    rel = 0.0
    if fin.any():
        rel = float((np.abs(got_lse[fin].astype(np.float64) - want_lse[fin]) / np.maximum(np.abs(want_lse[fin]), 1.0)).max())
    return err, rel, ok_inf


def _summary(errs, rels, infs, n):
    e = np.concatenate([x.reshape(-1) for x in errs]) if errs else np.zeros(1)
    return {"parity_checked_rows": n, "max_abs": float(e.max()), "mean_abs": float(e.mean()),
            "lse_rel": float(max(rels) if rels else 0.0), "lse_inf_pattern_ok": bool(all(infs)),
            "finite": bool(np.isfinite(e).all())}


def within_tolerance(s, max_abs=2e-2, mean_abs=2e-3, lse_rel=1e-3) -> bool:
    return s["finite"] and s["lse_inf_pattern_ok"] and s["max_abs"] <= max_abs and s["mean_abs"] <= mean_abs and s["lse_rel"] <= lse_rel


def pick_rows(lengths: torch.Tensor, count: int = 16):
    """First, last, longest, shortest and evenly spaced (row, token) pairs of a [B, s_q] length tensor."""
    B, s_q = lengths.shape
    flat = lengths.reshape(-1).cpu().numpy()
    n = flat.size
    chosen = {0, n - 1, int(flat.argmax()), int(flat.argmin())}
    for i in np.linspace(0, n - 1, max(count - len(chosen), 0) + 2).astype(int):
        chosen.add(int(i))
    return [(i // s_q, i % s_q) for i in sorted(chosen)][:max(count, 4)]


def check_csa_rows(q, kv_pool, block_table, indices, sm_scale, out, lse, rows, kv_len=None, topk_len=None, sink=None):
    errs, rels, infs = [], [], []
    sink_np = None if sink is None else sink.float().cpu().numpy()
    for b, j in rows:
        idx = indices[b, j].long()
        ok = idx >= 0
        if kv_len is not None:
            ok &= idx < int(kv_len[b, j])
        if topk_len is not None:
            ok &= torch.arange(idx.numel(), device=idx.device) < int(topk_len[b, j])
        idx = idx[ok]
        ent = kv_pool[block_table[b].long()[idx >> 6], idx & 63].cpu().numpy()
        o, l = orc.attend(q[b, j].float().cpu().numpy(), orc.unpack_entries(ent), sm_scale, sink_np)
        e, r, i = _compare(out[b, j].float().cpu().numpy(), lse[b, j].cpu().numpy(), orc.f32_to_bf16_bits(o), l)
        errs.append(e);  rels.append(r);  infs.append(i)
    return _summary(errs, rels, infs, len(rows))


def check_hca_rows(q, kv_pool, block_table, kv_len, win_pool, win_len, sm_scale, out, lse, rows, sink=None):
    errs, rels, infs = [], [], []
    sink_np = None if sink is None else sink.float().cpu().numpy()
    for b, j in rows:
        n, w = int(kv_len[b, j]), int(win_len[b, j])
        idx = torch.arange(n, device=q.device)
        ent = torch.cat([kv_pool[block_table[b].long()[idx >> 6], idx & 63], win_pool[b, :w]], 0).cpu().numpy()
        o, l = orc.attend(q[b, j].float().cpu().numpy(), orc.unpack_entries(ent), sm_scale, sink_np)
        e, r, i = _compare(out[b, j].float().cpu().numpy(), lse[b, j].cpu().numpy(), orc.f32_to_bf16_bits(o), l)
        errs.append(e);  rels.append(r);  infs.append(i)
    return _summary(errs, rels, infs, len(rows))
