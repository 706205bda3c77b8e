"""Allocation wrappers of the NVFP4 KEXT quantiser (masked residue channels appended along K).

Mirrors the public functions of the reference's csrc/nvfp4/quant.py:36-175: same names, argument
meaning, output shapes and errors.
"""
from __future__ import annotations

import torch

from .extension import ensure_loaded

# residue ratio -> selected channels per group of eight
_RATIO_TO_PER8 = {0.0: 0, 0.125: 1, 0.25: 2, 0.5: 4}


def _residue_per_8(num_salient: int, k: int) -> int:
    ratio = num_salient / k
    for known, per8 in _RATIO_TO_PER8.items():
        if abs(ratio - known) < 1e-3:
            return per8
    names = ", ".join(f"{r:.3f}" for r in sorted(_RATIO_TO_PER8))
    raise ValueError(
        f"Unsupported salient ratio {ratio:.4f} ({num_salient}/{k}). "
        f"Only the following ratios are supported: {names}.")


def indices_to_channel_masks(salient_indices: torch.Tensor, num_channels: int,
                             layer_name: str | None = None) -> torch.Tensor:
    """Channel indices -> uint8 [K/8]; bit b of byte g selects channel 8g+b."""
    del layer_name
    assert num_channels % 8 == 0, "num_channels must be multiple of 8"
    masks = torch.zeros(num_channels // 8, dtype=torch.uint8, device=salient_indices.device)
    bits = torch.bitwise_left_shift(torch.ones_like(salient_indices), salient_indices % 8).to(torch.uint8)
    masks.index_add_(0, salient_indices // 8, bits)
    return masks


def _quantize(x, input_scale, masks, num_salient, use_swapped_residue):
    m, k = x.shape
    per8 = _residue_per_8(num_salient, k)
    n_ext = k + num_salient
    codes = torch.empty(m * n_ext // 2, dtype=torch.uint8, device=x.device)
    scales = torch.empty(((m + 127) // 128) * ((n_ext + 63) // 64) * 512, dtype=torch.uint8, device=x.device)
    ensure_loaded()
    torch.ops.nvfp4.scaled_fp4_quant(codes, x, scales, input_scale, masks, n_ext, per8,
                                     use_swapped_residue)
    return codes.view(m, n_ext // 2), scales


def scaled_fp4_quant(input_tensor: torch.Tensor, input_scale: torch.Tensor,
                     salient_indices: torch.Tensor, use_swapped_residue: bool = False):
    """Quantize activations with residue channels selected by indices."""
    masks = indices_to_channel_masks(salient_indices, input_tensor.shape[1])
    return _quantize(input_tensor, input_scale, masks, len(salient_indices), use_swapped_residue)


def scaled_fp4_quant_with_mask(input_tensor: torch.Tensor, input_scale: torch.Tensor,
                               channel_masks: torch.Tensor, num_salient: int,
                               use_swapped_residue: bool = False):
    """FP4 quantization with pre-computed channel masks."""
    return _quantize(input_tensor, input_scale, channel_masks, num_salient, use_swapped_residue)


__all__ = ["indices_to_channel_masks", "scaled_fp4_quant", "scaled_fp4_quant_with_mask"]
