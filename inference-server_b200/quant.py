"""Load-time FP8 quantisation of expert weights (torch ops, any device).

Weights are cut into 128x128 tiles; each tile gets scale = 448 / amax (1 for an
all-zero tile), q = clamp(w * scale, +-448) rounded to e4m3, and the stored
factor is scale_inv = 1 / scale, so w ~= q * scale_inv.  This is the block-scale
convention of the FP8 checkpoints the reference's model loader consumes
(transformers finegrained FP8: weight + weight_scale_inv).  It runs once when
weights are loaded and is not part of the per-step path.
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
BLOCK = 128


def quantize_weight_blocks(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w [..., rows, cols] (rows, cols multiples of 128) -> (e4m3 same shape,
    scale_inv fp32 [..., rows/128, cols/128])."""
    rows, cols = w.shape[-2], w.shape[-1]
    if rows % BLOCK or cols % BLOCK:
        raise ValueError(f"weight shape ({rows}, {cols}) is not a multiple of {BLOCK}")
    lead = w.shape[:-2]
    t = w.to(torch.float32).reshape(*lead, rows // BLOCK, BLOCK, cols // BLOCK, BLOCK)
    amax = t.abs().amax(dim=(-3, -1))
    scale = torch.where(amax > 0, FP8_MAX / torch.where(amax > 0, amax, torch.ones_like(amax)),
                        torch.ones_like(amax))
    q = (t * scale.unsqueeze(-1).unsqueeze(-3)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(w.shape), (1.0 / scale).to(torch.float32)


def dequantize_weight_blocks(q: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """Inverse of quantize_weight_blocks, fp32."""
    rows, cols = q.shape[-2], q.shape[-1]
    lead = q.shape[:-2]
    t = q.to(torch.float32).reshape(*lead, rows // BLOCK, BLOCK, cols // BLOCK, BLOCK)
    return (t * scale_inv.unsqueeze(-1).unsqueeze(-3)).reshape(q.shape)


def tile_weight_blocks(q: torch.Tensor) -> torch.Tensor:
    """[..., rows, cols] -> [..., rows/128, cols/128, 128, 128]: every 128x128 block contiguous (16 KiB
    of e4m3), the layout the grouped GEMM streams fastest (one sequential read per TMA box)."""
    rows, cols = q.shape[-2], q.shape[-1]
    lead = q.shape[:-2]
    return q.reshape(*lead, rows // BLOCK, BLOCK, cols // BLOCK, BLOCK).transpose(-3, -2).contiguous()


def untile_weight_blocks(t: torch.Tensor) -> torch.Tensor:
    """Inverse of tile_weight_blocks."""
    rb, cb = t.shape[-4], t.shape[-3]
    lead = t.shape[:-4]
    return t.transpose(-3, -2).reshape(*lead, rb * BLOCK, cb * BLOCK).contiguous()
