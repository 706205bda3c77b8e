"""Python API of the NVFP4 kernels, under the names of the reference's ``nvfp4`` wheel
(ShawRong/ResInfer csrc/nvfp4/__init__.py:5-19)."""
from .extension import ensure_loaded
from .mext import scaled_fp4_quant_mext_r1
from .quant import indices_to_channel_masks, scaled_fp4_quant, scaled_fp4_quant_with_mask
from .scale_layout import swizzle_scales

__all__ = [
    "ensure_loaded",
    "indices_to_channel_masks",
    "scaled_fp4_quant",
    "scaled_fp4_quant_mext_r1",
    "scaled_fp4_quant_with_mask",
    "swizzle_scales",
]
