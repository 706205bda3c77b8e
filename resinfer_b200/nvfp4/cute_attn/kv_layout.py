"""Typed view of a stock NVFP4 paged KV cache, as consumed by ResAttn decode.

Same fields as the reference's NvFp4PagedKVPool (csrc/resattn/kv_layout.py:16-28).  The reference
kernel supports page size 128 only; this library takes any multiple of 16, so ``page_size`` is a real
parameter here (default 128 for drop-in use).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

SF_VEC = 16
PAGE_SIZE = 128


@dataclass
class NvFp4PagedKVPool:
    """k_data / v_data: uint8 [pages, Hkv, page_size, D/2]; k_sf / v_sf: E4M3 bytes
    [pages, Hkv, page_size, D/16]; the global scales multiply the dequantised K / V."""
    num_kv_heads: int
    head_dim: int
    k_data: torch.Tensor
    v_data: torch.Tensor
    k_sf: torch.Tensor
    v_sf: torch.Tensor
    page_size: int = PAGE_SIZE
    k_global_scale: float = 1.0
    v_global_scale: float = 1.0
    layout_profile: ClassVar[str] = "trtllm"
