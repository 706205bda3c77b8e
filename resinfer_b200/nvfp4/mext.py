"""Allocation wrapper of the NVFP4 MEXT quantiser (base + full-channel residue).

Mirrors ``scaled_fp4_quant_mext_r1`` of the reference (csrc/nvfp4/mext.py:97-192): keyword
names, environment defaults (NVFP4_MEXT_R1_ELTS_PER_THREAD, RESIDUE_MEXT_R1_LAYOUT,
NVFP4_MEXT_R1_PDL), output shapes and ValueErrors.
"""
from __future__ import annotations

import os

import torch

from .extension import ensure_loaded

LAYOUT_CONCAT, LAYOUT_ROW_PAIR, LAYOUT_TILE8, LAYOUT_CONCAT_K, LAYOUT_ATTN_TILE8 = range(5)

_LAYOUT_NAMES = {
    LAYOUT_CONCAT: ("", "concat", "default", "base_residue"),
    LAYOUT_ROW_PAIR: ("row_pair", "rowpair", "pair", "interleaved"),
    LAYOUT_TILE8: ("tile8", "tile_8", "tile8_pair", "tile8_row_pair"),
    LAYOUT_ATTN_TILE8: ("attn_tile8", "attention_tile8", "qk_tile8", "gqa_tile8"),
    LAYOUT_CONCAT_K: ("concat_k", "kext", "k_concat", "kloop"),
}
_ELTS_NAMES = {0: ("", "auto", "default"), 8: ("8", "elts8", "elts_8"), 16: ("16", "elts16", "elts_16")}


def _lookup(value, table, env, default, what, expected):
    if value is None:
        value = os.getenv(env, default)
    if isinstance(value, str):
        key = value.strip().lower().replace("-", "_")
        for code, names in table.items():
            if key in names:
                return code
        raise ValueError(f"Unsupported mext_r1 {what} '{value}'. Expected one of: {expected}.")
    if value in table:
        return int(value)
    raise ValueError(f"Unsupported mext_r1 {what} {value!r}. Expected one of: {expected}.")


def _resolve_pdl(enable_pdl, device) -> bool:
    if enable_pdl is not None:
        return bool(enable_pdl)
    configured = os.getenv("NVFP4_MEXT_R1_PDL", "auto").strip().lower()
    if configured in ("1", "true", "on", "yes"):
        return True
    if configured in ("0", "false", "off", "no"):
        return False
    if configured in ("", "auto", "default"):
        return torch.cuda.get_device_capability(device)[0] >= 9
    raise ValueError(f"NVFP4_MEXT_R1_PDL must be auto/on/off (or 1/0), got {configured!r}")


def scaled_fp4_quant_mext_r1(input_tensor: torch.Tensor, input_scale: torch.Tensor, *,
                             elts_mode=None, layout_mode=None, m_pad_multiple=None,
                             enable_pdl: bool | None = None):
    """Quantize activations and their full-channel residue into packed FP4 outputs.

    Returns ``(codes, scales)``: codes uint8 [2*M', K/2] (``[M, K]`` bytes for concat_k), scales
    the flat 128x4-swizzled E4M3 buffer of the layout."""
    elts = _lookup(elts_mode, _ELTS_NAMES, "NVFP4_MEXT_R1_ELTS_PER_THREAD", "auto", "elts_mode", "auto, 8, 16")
    layout = _lookup(layout_mode, _LAYOUT_NAMES, "RESIDUE_MEXT_R1_LAYOUT", "concat", "layout_mode",
                     "concat, row_pair, tile8, attn_tile8, concat_k")
    pdl = _resolve_pdl(enable_pdl, input_tensor.device)
    m, k = input_tensor.shape
    if k % 16:
        raise ValueError(f"scaled_fp4_quant_mext_r1 requires K multiple of 16, got {k}")
    tile8 = layout in (LAYOUT_TILE8, LAYOUT_ATTN_TILE8)
    if m_pad_multiple is None:
        if tile8 and m % 8:
            raise ValueError("tile8 layouts require M to be divisible by 8, "
                             "or pass m_pad_multiple=8 to request padded row+8 output.")
        out_m = m
    else:
        if not tile8:
            raise ValueError("m_pad_multiple is supported only with tile8 layouts")
        pad = int(m_pad_multiple)
        if pad <= 0:
            raise ValueError(f"m_pad_multiple must be positive, got {pad}")
        out_m = -(-m // pad) * pad
    dev = input_tensor.device
    codes = torch.empty(out_m * k, dtype=torch.uint8, device=dev)
    k_tiles = (k + 63) // 64
    if layout == LAYOUT_CONCAT_K:
        n_scale = ((out_m + 127) // 128) * ((2 * k + 63) // 64) * 512
        scales = torch.empty(n_scale, dtype=torch.uint8, device=dev)
    elif layout == LAYOUT_ATTN_TILE8:
        # one private 128-row scale tile per 8 tokens; rows the kernel never touches must read 0
        scales = torch.zeros((out_m // 8) * k_tiles * 512, dtype=torch.uint8, device=dev)
    else:
        scales = torch.empty(((2 * out_m + 127) // 128) * k_tiles * 512, dtype=torch.uint8, device=dev)
    ensure_loaded()
    torch.ops.nvfp4.scaled_fp4_quant_mext_r1(codes, input_tensor, scales, input_scale, elts, layout, pdl)
    if layout == LAYOUT_CONCAT_K:
        return codes.view(out_m, k), scales
    return codes.view(2 * out_m, k // 2), scales


__all__ = ["scaled_fp4_quant_mext_r1"]
