"""Scale-layout helpers shared by the vLLM linear methods (reference: quant/vllm_integration/util.py:16-34)."""
from __future__ import annotations

import torch
from torch.nn.parameter import Parameter

from ..weight_prep import swizzle_scales_any


def swizzle_blockscale(scale: torch.Tensor) -> torch.Tensor:
    """E4M3 block scales [N, K/16] (float8_e4m3fn or their bytes) -> the 128x4-swizzled buffer the GEMM reads,
    as float8_e4m3fn [ceil(N/128)*128, ceil(K/64)*4] (zero padded)."""
    if scale.ndim != 2:
        raise ValueError(f"block scales must be 2-D, got {tuple(scale.shape)}")
    raw = scale.view(torch.uint8) if scale.dtype == torch.float8_e4m3fn else scale
    if raw.dtype != torch.uint8:
        raise ValueError("block scales must be float8_e4m3fn (or their uint8 bytes)")
    rows = (scale.shape[0] + 127) // 128 * 128
    cols = (scale.shape[1] + 3) // 4 * 4
    return swizzle_scales_any(raw.contiguous()).view(torch.float8_e4m3fn).reshape(rows, cols)


def prepare_decode_mext_scale(layer, raw_weight_scale_ext: torch.Tensor) -> None:
    """Base-K scale buffer of a K-extended layer for the fold route: the first K_base / 16 groups of the RAW
    checkpoint scale, swizzled on their own (a swizzled buffer over K + S cannot be sliced).  The packed weight
    is shared: the fold GEMM reads its base-K prefix through the row stride."""
    k_base = int(layer.original_in_features)
    if k_base <= 0 or k_base % 16:
        raise ValueError(f"base K must be a positive multiple of 16, got {k_base}")
    if raw_weight_scale_ext.ndim != 2 or raw_weight_scale_ext.shape[1] < k_base // 16 or k_base > layer.weight.shape[1] * 2:
        raise ValueError("extended scale / weight narrower than the base K")
    layer.weight_scale_base = Parameter(swizzle_blockscale(raw_weight_scale_ext[:, :k_base // 16].contiguous()),
                                        requires_grad=False)
    layer._mext_decode_k_base = k_base
    layer._decode_mext_layout_enabled = True
