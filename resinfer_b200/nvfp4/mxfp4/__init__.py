"""MXFP4 quantisers and GEMMs under the reference's ``nvfp4.mxfp4`` names
(ShawRong/ResInfer csrc/mxfp4/__init__.py:5-18)."""
from ..scale_layout import swizzle_scales
from .dense import fold_gemm, gemm
from .quantization import quantize, quantize_mext
from .selective import prepare_indices, quantize_selective

__all__ = ["quantize", "quantize_mext", "swizzle_scales", "gemm", "fold_gemm", "prepare_indices",
           "quantize_selective"]
