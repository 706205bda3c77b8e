"""Registers the native torch ops ``nvfp4::*`` on top of the C-ABI library.

Same four schemas as the reference's TORCH_LIBRARY block
(ShawRong/ResInfer csrc/bindings/pybind.cpp:28-54), CUDA dispatch key only, caller-allocated
outputs mutated in place, launched on the current stream of the input's device, no host
synchronisation.  ``ensure_loaded`` mirrors csrc/nvfp4/extension.py:56-83, except that a missing
library is an error as soon as an op is needed: there is no fallback path.
"""
from __future__ import annotations

import warnings

import torch

from .. import _cabi

_LOADED = False
_LIB = None

_MISSING_MSG = (
    "resinfer_b200 native library not found or unloadable. Build it with "
    "`python -m resinfer_b200.build`. The NVFP4/MXFP4 quantisers, the FP4 GEMM and ResAttn "
    "decode require this library."
)

_SCHEMAS = {
    "scaled_fp4_quant":
        "(Tensor(a!) output, Tensor input, Tensor(b!) output_scale, Tensor input_scale, "
        "Tensor channel_indices, int n_ext, int residue_per_8, bool use_swapped_residue) -> ()",
    "scaled_fp4_quant_mext_r1":
        "(Tensor(a!) output, Tensor input, Tensor(b!) output_scale, Tensor input_scale, "
        "int elts_mode, int layout_mode, bool enable_pdl=True) -> ()",
    "scaled_fp4_quant_mext_r1_grouped_q":
        "(Tensor q, Tensor(a!) q_pack, Tensor(b!) q_sf) -> ()",
    "mxfp4_residue_quant":
        "(Tensor x, Tensor(a!) q, Tensor(b!) sf, Tensor? masks, int per8, bool swizzle, "
        "bool tile8=False, int pdl_mode=0) -> ()",
}


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _scaled_fp4_quant(output, input, output_scale, input_scale, channel_indices, n_ext,
                      residue_per_8, use_swapped_residue):
    _require(input.dim() == 2 and input.stride(1) == 1, "input must be [M, K] with unit column stride")
    m, k = input.shape
    with torch.cuda.device(input.device):
        st = _LIB.ri_nvfp4_quant_kext(
            input.data_ptr(), _cabi.torch_dtype_code(input.dtype), m, k, input.stride(0),
            input_scale.data_ptr(), channel_indices.data_ptr(), int(residue_per_8), int(n_ext),
            output.data_ptr(), output.numel() * output.element_size(),
            output_scale.data_ptr(), output_scale.numel() * output_scale.element_size(),
            int(bool(use_swapped_residue)), _cabi.current_stream(input.device))
    _cabi.check(st, "nvfp4::scaled_fp4_quant")


def _scaled_fp4_quant_mext_r1(output, input, output_scale, input_scale, elts_mode, layout_mode,
                              enable_pdl=True):
    # elts_mode selected between two thread decompositions of the reference kernel; both give the
    # same bytes, this library has one decomposition and ignores the value (after validating it).
    _require(int(elts_mode) in (0, 8, 16), "elts_mode must be 0 (auto), 8 or 16")
    _require(input.dim() == 2 and input.stride(1) == 1, "input must be [M, K] with unit column stride")
    m, k = input.shape
    layout = int(layout_mode) if int(layout_mode) in (0, 1, 2, 3, 4, 5) else 0   # unknown -> concat
    with torch.cuda.device(input.device):
        st = _LIB.ri_nvfp4_quant_mext(
            input.data_ptr(), _cabi.torch_dtype_code(input.dtype), m, k, input.stride(0),
            input_scale.data_ptr(), input_scale.numel(),
            output.data_ptr(), output.numel() * output.element_size(),
            output_scale.data_ptr(), output_scale.numel() * output_scale.element_size(),
            layout, int(bool(enable_pdl)), _cabi.current_stream(input.device))
    _cabi.check(st, "nvfp4::scaled_fp4_quant_mext_r1")


def _grouped_q(q, q_pack, q_sf):
    _require(q.is_cuda and q_pack.is_cuda and q_sf.is_cuda and q.device == q_pack.device == q_sf.device,
             "grouped Q tensors must share one CUDA device")
    _require(q.dtype == torch.bfloat16 and q.is_contiguous() and q.dim() == 4,
             "q must be contiguous BF16 [B, Hkv, G, D]")
    _require(q_pack.dtype == torch.uint8 and q_sf.dtype == torch.uint8 and q_pack.is_contiguous()
             and q_sf.is_contiguous(), "grouped Q outputs must be contiguous uint8")
    b, h, g, d = q.shape
    _require(g in (4, 6, 8), "grouped residue Q supports GQA4/6/8")
    _require(d in (128, 256), "grouped residue Q requires head_dim=128 or 256")
    p = 8 if g == 4 else 16
    _require(tuple(q_pack.shape) == (b, h, p, d // 2), "q_pack shape must match the physical Q tile")
    with torch.cuda.device(q.device):
        st = _LIB.ri_nvfp4_quant_grouped_q(q.data_ptr(), b, h, g, d, q_pack.data_ptr(), q_pack.numel(),
                                           q_sf.data_ptr(), q_sf.numel(), _cabi.current_stream(q.device))
    _cabi.check(st, "nvfp4::scaled_fp4_quant_mext_r1_grouped_q")


def _mxfp4_residue_quant(x, q, sf, masks, per8, swizzle, tile8=False, pdl_mode=0):
    _require(x.is_cuda and x.dim() == 2, "expected CUDA [M,K]")
    _require(x.dtype in (torch.float16, torch.bfloat16), "fp16/bf16 required")
    _require(q.is_cuda and sf.is_cuda and q.device == x.device and sf.device == x.device,
             "output device mismatch")
    _require(q.dtype == torch.uint8 and sf.dtype == torch.uint8 and q.is_contiguous() and sf.is_contiguous(),
             "contiguous uint8 outputs required")
    m, k = x.shape
    if masks is not None:
        _require(masks.device == x.device and masks.dtype == torch.uint8 and masks.is_contiguous()
                 and masks.dim() == 1 and masks.numel() == k // 8, "prepared uint8 masks [K/8] required")
    _require(q.dim() == 2, "invalid output rows")
    with torch.cuda.device(x.device):
        st = _LIB.ri_mxfp4_quant(
            x.data_ptr(), _cabi.torch_dtype_code(x.dtype), m, k, x.stride(0), x.stride(1),
            _cabi.ptr(masks), int(per8), q.data_ptr(), q.shape[0], q.shape[1],
            sf.data_ptr(), sf.numel(), int(bool(swizzle)), int(bool(tile8)), int(pdl_mode),
            _cabi.current_stream(x.device))
    _cabi.check(st, "nvfp4::mxfp4_residue_quant")


_IMPLS = {
    "scaled_fp4_quant": _scaled_fp4_quant,
    "scaled_fp4_quant_mext_r1": _scaled_fp4_quant_mext_r1,
    "scaled_fp4_quant_mext_r1_grouped_q": _grouped_q,
    "mxfp4_residue_quant": _mxfp4_residue_quant,
}

_torch_lib = None


def ensure_loaded(required: bool = True) -> bool:
    """Load the C-ABI library and register the ``nvfp4::*`` ops.  Returns whether the operators
    are available; raises ImportError when ``required`` and they are not."""
    global _LOADED, _LIB, _torch_lib
    if _LOADED:
        return True
    try:
        _LIB = _cabi.load()
    except (ImportError, OSError, AttributeError) as exc:
        if required:
            raise ImportError(_MISSING_MSG) from exc
        warnings.warn(f"{_MISSING_MSG} ({exc})", RuntimeWarning, stacklevel=2)
        return False
    _torch_lib = torch.library.Library("nvfp4", "DEF")
    for name, schema in _SCHEMAS.items():
        _torch_lib.define(name + schema)
        _torch_lib.impl(name, _IMPLS[name], "CUDA")
    _LOADED = True
    return True


ensure_loaded(required=False)

__all__ = ["ensure_loaded"]
