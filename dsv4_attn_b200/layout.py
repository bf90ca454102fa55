"""Cache-entry layout helpers (torch, any device): quantise and pack BF16/FP32
latent + RoPE rows into the 656-byte entry the kernels read, and the inverse.

Entry: 512 FP8 e4m3 latent | 4 FP32 scales (one per 128 latent elements,
scale = absmax / 448, the reference quantiser's recipe of
bench/bench/decode.py:92-114 with an FP32 scale) | 64 BF16 RoPE values."""
from __future__ import annotations

import torch

D_LATENT = 512
D_ROPE = 64
D_QK = 576
SCALE_BLOCK = 128
N_SCALES = 4
SCALE_OFF = 512
ROPE_OFF = 528
ENTRY_BYTES = 656
PAGE_ENTRIES = 64
PAGE_BYTES = PAGE_ENTRIES * ENTRY_BYTES


def pack_entries(latent: torch.Tensor, rope: torch.Tensor) -> torch.Tensor:
    """latent [..., 512], rope [..., 64] (float32 or bf16) -> uint8 [..., 656]."""
    if latent.shape[-1] != D_LATENT or rope.shape[-1] != D_ROPE or latent.shape[:-1] != rope.shape[:-1]:
        raise ValueError(f"expected [..., 512] and [..., 64], got {tuple(latent.shape)} {tuple(rope.shape)}")
    lead = latent.shape[:-1]
    blk = latent.float().reshape(*lead, N_SCALES, SCALE_BLOCK)
    scale = blk.abs().amax(dim=-1) / 448.0
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = (blk / scale.unsqueeze(-1)).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
    out = torch.empty(*lead, ENTRY_BYTES, dtype=torch.uint8, device=latent.device)
    out[..., :D_LATENT] = q.view(torch.uint8).reshape(*lead, D_LATENT)
    out[..., SCALE_OFF:ROPE_OFF] = scale.contiguous().view(torch.uint8).reshape(*lead, 4 * N_SCALES)
    out[..., ROPE_OFF:] = rope.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(*lead, 2 * D_ROPE)
    return out


def unpack_entries(entries: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 656] -> float32 [..., 576] (exact dequantisation)."""
    lead = entries.shape[:-1]
    lat = entries[..., :D_LATENT].contiguous().view(torch.float8_e4m3fn).float()
    scale = entries[..., SCALE_OFF:ROPE_OFF].contiguous().view(torch.float32)
    lat = (lat.reshape(*lead, N_SCALES, SCALE_BLOCK) * scale.reshape(*lead, N_SCALES, 1)).reshape(*lead, D_LATENT)
    rope = entries[..., ROPE_OFF:].contiguous().view(torch.bfloat16).float().reshape(*lead, D_ROPE)
    return torch.cat([lat, rope], dim=-1)
