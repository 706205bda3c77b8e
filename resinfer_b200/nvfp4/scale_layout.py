"""The 128x4 byte-scale layout shared by the NVFP4 and MXFP4 operators.

Byte offset of the scale of (row m, k-group g):
    (m // 128) * (ceil(G / 4) * 512) + (g // 4) * 512 + (m % 32) * 16 + ((m % 128) // 32) * 4 + g % 4
which is the layout tcgen05.cp copies into tensor memory unchanged.  Same result as the
reference's ``swizzle_scales`` (ShawRong/ResInfer csrc/nvfp4/scale_layout.py:8-33).
"""
from __future__ import annotations

import torch


def swizzle_scales(scales: torch.Tensor) -> torch.Tensor:
    """uint8 [M, G] or [B, M, G] linear scales -> flat (per batch) swizzled buffer, zero padded to
    128 rows x 4 groups."""
    if (scales.ndim not in (2, 3) or scales.dtype != torch.uint8 or not scales.is_cuda
            or not scales.is_contiguous()):
        raise ValueError("expected contiguous CUDA uint8 [M,G] or [B,M,G] scales")
    rows, groups = scales.shape[-2:]
    if groups <= 0:
        raise ValueError("scale K extent must be nonempty")
    batched = scales.ndim == 3
    nb = scales.shape[0] if batched else 1
    row_tiles, k_tiles = (rows + 127) // 128, (groups + 3) // 4
    # destination viewed as [batch, row_tile, k_tile, m%32, (m%128)//32, g%4]
    out = torch.zeros((nb, row_tiles, k_tiles, 32, 4, 4), dtype=torch.uint8, device=scales.device)
    m = torch.arange(rows, device=scales.device)
    g = torch.arange(groups, device=scales.device)
    out[:, (m // 128)[:, None], (g // 4)[None, :], (m % 32)[:, None], ((m % 128) // 32)[:, None],
        (g % 4)[None, :]] = scales.reshape(nb, rows, groups)
    out = out.reshape(nb, -1)
    return out if batched else out[0]


__all__ = ["swizzle_scales"]
