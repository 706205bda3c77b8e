"""MXFP4 activation quantisation (32-element blocks, E8M0 scale = smallest power of two >= amax/6).

Public names and errors follow the reference's csrc/mxfp4/quantization.py:51-78 and
csrc/mxfp4/residue_quant.py:16-71.  ``quantize`` (no residue) runs this library's own kernel; the
reference delegates that one to FlashInfer.
"""
from __future__ import annotations

import torch

from ..extension import ensure_loaded

_PDL_MODES = {"off": 0, "tail": 1, "early": 2}


def _ceildiv(a: int, b: int) -> int:
    return -(-a // b)


def _check_recipe(recipe: str) -> None:
    if recipe != "ceil":
        raise ValueError("MXFP4 uses vLLM/FlashInfer native ceil quantization; legacy ocp is unsupported")


def _validate_2d(source: torch.Tensor, layout: str, recipe: str) -> int:
    _check_recipe(recipe)
    if source.ndim != 2 or not source.is_cuda or source.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("expected CUDA fp16/bf16 [M,K]")
    k = source.shape[1]
    if k <= 0 or k % 32:
        raise ValueError("K must be a positive multiple of 32")
    if layout not in ("linear", "128x4"):
        raise ValueError("layout must be linear or 128x4")
    return k


def _alloc_scales(rows: int, k_total: int, layout: str, device) -> torch.Tensor:
    if layout == "linear":
        return torch.empty((rows, k_total // 32), device=device, dtype=torch.uint8)
    return torch.empty((_ceildiv(rows, 128) * _ceildiv(k_total, 128) * 512,), device=device, dtype=torch.uint8)


def quantize_residue(source, *, masks=None, per8=0, layout="linear", kp=None, mext_layout="row_pair",
                     m_pad_multiple=None, pdl_mode="off"):
    """Quantise ``source`` plus its residue: all channels (``masks`` None, two output rows per input
    row) or the channels selected by ``masks`` (appended along K, zero padded to ``kp``)."""
    _validate_2d(source, layout, "ceil")
    if pdl_mode not in _PDL_MODES:
        raise ValueError("pdl_mode must be off, tail or early")
    if mext_layout not in ("row_pair", "tile8"):
        raise ValueError("mext_layout must be row_pair or tile8")
    rows, k = source.shape
    k_total = k if kp is None else kp
    tile8 = mext_layout == "tile8"
    if tile8:
        if masks is not None or layout != "128x4":
            raise ValueError("tile8 requires full residue and 128x4 scales")
        pad = 8 if m_pad_multiple is None else int(m_pad_multiple)
        if pad <= 0 or pad % 8:
            raise ValueError("tile8 m_pad_multiple must be a positive multiple of 8")
        out_m = _ceildiv(rows, pad) * pad
    else:
        if m_pad_multiple is not None:
            raise ValueError("m_pad_multiple is supported only for tile8")
        out_m = rows
    out_rows = out_m * (2 if masks is None else 1)
    packed = torch.empty((out_rows, k_total // 2), device=source.device, dtype=torch.uint8)
    scales = _alloc_scales(out_rows, k_total, layout, source.device)
    if rows:
        ensure_loaded()
        torch.ops.nvfp4.mxfp4_residue_quant(source, packed, scales, masks, per8, layout == "128x4", tile8,
                                            _PDL_MODES[pdl_mode])
    return packed, scales


def quantize(source, *, layout="128x4", recipe="ceil"):
    """Plain MXFP4 quantisation: codes [M, K/2] and scales (128x4-swizzled flat, or linear [M, K/32])."""
    k = _validate_2d(source, layout, recipe)
    rows = source.shape[0]
    packed = torch.empty((rows, k // 2), device=source.device, dtype=torch.uint8)
    if layout == "linear":
        scales = torch.empty((rows, k // 32), device=source.device, dtype=torch.uint8)
    else:
        scales = torch.empty((_ceildiv(rows, 128) * _ceildiv(k, 128) * 512,) if rows else (0,),
                             device=source.device, dtype=torch.uint8)
    if rows:
        ensure_loaded()
        torch.ops.nvfp4.mxfp4_residue_quant(source, packed, scales, None, 0, layout == "128x4", False, 0)
    return packed, scales


def quantize_mext(source, *, layout="128x4", recipe="ceil", mext_layout="row_pair", m_pad_multiple=None,
                  pdl_mode="off"):
    """Quantize activations and their full-channel residue."""
    _check_recipe(recipe)
    return quantize_residue(source, layout=layout, mext_layout=mext_layout, m_pad_multiple=m_pad_multiple,
                            pdl_mode=pdl_mode)
