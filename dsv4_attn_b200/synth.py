"""Seeded synthetic decode workloads built directly on the device (torch).

Values are N(0,1) as the benchmark configurations state: q BF16, latent
quantised to FP8 e4m3 with one FP32 absmax scale per 128 elements, RoPE tail
BF16, pages of 64 entries behind a random block table, top-k index lists of
distinct uniform indices with -1 padding where the visible context is shorter
than top-k.  No dataset is involved."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence, Union

import torch

from .layout import D_LATENT, D_QK, D_ROPE, ENTRY_BYTES, PAGE_ENTRIES, pack_entries

IntOrSeq = Union[int, Sequence[int]]


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def random_pool(num_pages: int, device, g, chunk_pages: int = 1024) -> torch.Tensor:
    pool = torch.empty(num_pages, PAGE_ENTRIES, ENTRY_BYTES, dtype=torch.uint8, device=device)
    for p0 in range(0, num_pages, chunk_pages):
        n = min(chunk_pages, num_pages - p0)
        lat = torch.randn(n, PAGE_ENTRIES, D_LATENT, generator=g, device=device)
        rope = torch.randn(n, PAGE_ENTRIES, D_ROPE, generator=g, device=device)
        pool[p0:p0 + n] = pack_entries(lat, rope)
    return pool


def _block_table(pages_per: torch.Tensor, g, device):
    B = pages_per.numel()
    max_pages = int(pages_per.max().item())
    P = int(pages_per.sum().item())
    perm = torch.randperm(P, generator=g, device=device).to(torch.int32)
    bt = torch.zeros(B, max_pages, dtype=torch.int32, device=device)
    off = 0
    for b, n in enumerate(pages_per.tolist()):
        bt[b, :n] = perm[off:off + n]
        off += n
    return bt, P


@dataclass
class CsaWorkload:
    q: torch.Tensor
    kv_pool: torch.Tensor
    block_table: torch.Tensor
    indices: torch.Tensor
    kv_len: torch.Tensor
    topk_len: torch.Tensor      # [B, s_q] leading index slots in use
    sm_scale: float
    valid_entries: int          # sum over (request, token) of gathered entries

    @property
    def kv_bytes(self) -> int:
        return self.valid_entries * ENTRY_BYTES


def make_csa(seed: int, B: int, s_q: int, H: int, n_entries: IntOrSeq, topk: int, device="cuda") -> CsaWorkload:
    g = _gen(device, seed)
    n_ent = torch.as_tensor([n_entries] * B if isinstance(n_entries, int) else list(n_entries), dtype=torch.int64)
    pages_per = torch.clamp((n_ent + PAGE_ENTRIES - 1) // PAGE_ENTRIES, min=1)
    q = torch.randn(B, s_q, H, D_QK, generator=g, device=device).to(torch.bfloat16)
    bt, P = _block_table(pages_per, g, device)
    pool = random_pool(P, device, g)
    indices = torch.full((B, s_q, topk), -1, dtype=torch.int32, device=device)
    kv_len = torch.zeros(B, s_q, dtype=torch.int32)
    topk_len = torch.zeros(B, s_q, dtype=torch.int32)
    valid = 0
    for b in range(B):
        for j in range(s_q):
            vis = max(int(n_ent[b]) - (s_q - 1 - j), 0)
            kv_len[b, j] = vis
            k = min(topk, vis)
            topk_len[b, j] = k
            if k > 0:
                indices[b, j, :k] = torch.randperm(vis, generator=g, device=device)[:k].to(torch.int32)
            valid += k
    return CsaWorkload(q, pool, bt, indices, kv_len.to(device), topk_len.to(device), 1.0 / math.sqrt(D_QK), valid)


@dataclass
class HcaWorkload:
    q: torch.Tensor
    kv_pool: torch.Tensor
    block_table: torch.Tensor
    kv_len: torch.Tensor
    win_pool: torch.Tensor
    win_len: torch.Tensor
    attn_sink: Optional[torch.Tensor]
    sm_scale: float
    valid_entries: int
    max_len: int

    @property
    def kv_bytes(self) -> int:
        return self.valid_entries * ENTRY_BYTES


def make_hca(seed: int, B: int, s_q: int, H: int, kv_len: IntOrSeq, win_len: IntOrSeq, W: int = 128,
             with_sink: bool = False, device="cuda") -> HcaWorkload:
    g = _gen(device, seed)
    kvl = torch.as_tensor([kv_len] * B if isinstance(kv_len, int) else list(kv_len), dtype=torch.int64)
    wl = torch.as_tensor([win_len] * B if isinstance(win_len, int) else list(win_len), dtype=torch.int64)
    pages_per = torch.clamp((kvl + PAGE_ENTRIES - 1) // PAGE_ENTRIES, min=1)
    q = torch.randn(B, s_q, H, D_QK, generator=g, device=device).to(torch.bfloat16)
    bt, P = _block_table(pages_per, g, device)
    pool = random_pool(P, device, g)
    win = pack_entries(torch.randn(B, W, D_LATENT, generator=g, device=device),
                       torch.randn(B, W, D_ROPE, generator=g, device=device))
    sink = (torch.randn(H, generator=g, device=device) * 0.5) if with_sink else None
    kv2 = kvl[:, None].repeat(1, s_q).to(torch.int32)
    w2 = torch.stack([torch.clamp(wl - (s_q - 1 - j), min=0) for j in range(s_q)], dim=1).to(torch.int32)
    valid = int((kv2.long() + w2.long()).sum().item())
    max_len = int((kv2.long() + w2.long()).max().item())
    return HcaWorkload(q, pool, bt, kv2.to(device), win, w2.to(device), sink, 1.0 / math.sqrt(D_QK), valid, max_len)


def lognormal_contexts(n: int, seed: int = 0, median: int = 8192, sigma: float = 1.0,
                       lo: int = 1024, hi: int = 131072) -> list[int]:
    """Per-request raw context lengths for the mixed workload: log-normal with
    the given median, clipped to [lo, hi]."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g) * sigma + math.log(median)
    return torch.clamp(torch.exp(x), lo, hi).round().to(torch.int64).tolist()


def make_mixed(seed: int, contexts: Sequence[int], H: int = 128, topk: int = 2048, device="cuda"):
    """The two layers of the mixed decode workload for one shard of requests:
    a CSA layer (compression ratio 4: ctx // 4 entries, top-k `topk`) and an HCA
    layer (ratio 128: ctx // 128 entries plus a 128-entry window)."""
    csa = make_csa(seed, len(contexts), 1, H, [max(c // 4, 1) for c in contexts], topk, device=device)
    hca = make_hca(seed + 1, len(contexts), 1, H, [c // 128 for c in contexts], [min(128, c) for c in contexts],
                   device=device)
    return csa, hca
