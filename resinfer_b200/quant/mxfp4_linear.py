"""``residue::mxfp4_linear`` -- the opaque MXFP4 linear op.

Schema, modes ("standard", "selective", "mext_r1"), errors and fake implementation follow the
reference's quant/mxfp4_linear.py:9-76.
"""
from __future__ import annotations

import torch


def mxfp4_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, indices: torch.Tensor,
                 masks: torch.Tensor, mode: str, output_dtype: torch.dtype,
                 bias: torch.Tensor | None = None) -> torch.Tensor:
    from ..nvfp4.mxfp4 import fold_gemm, gemm, quantize, quantize_mext, quantize_selective
    if mode not in ("standard", "selective", "mext_r1"):
        raise ValueError(f"unknown MXFP4 linear mode {mode}")
    if x.ndim < 1 or x.shape[-1] == 0:
        raise ValueError("linear input must have a positive feature dimension")
    if x.device.type != "cuda" or torch.cuda.get_device_capability(x.device)[0] != 10:
        raise ValueError("MXFP4 linear currently requires SM100")
    out_shape = (*x.shape[:-1], weight.shape[0])
    rows = x.numel() // x.shape[-1]
    if rows == 0:
        return torch.empty(out_shape, device=x.device, dtype=output_dtype)
    src = x.reshape(rows, x.shape[-1])
    if mode == "mext_r1":
        act, act_sf = quantize_mext(src, pdl_mode="early")
        out = fold_gemm(act, weight, act_sf, weight_scale, out_dtype=output_dtype)
    else:
        act, act_sf = quantize_selective(src, indices, masks) if mode == "selective" else quantize(src)
        out = gemm(act, weight, act_sf, weight_scale, out_dtype=output_dtype)
    if bias is not None:
        out = (out + bias).to(output_dtype)
    return out.reshape(out_shape)


def _fake_mxfp4_linear(x, weight, weight_scale, indices, masks, mode, output_dtype, bias=None):
    return torch.empty((*x.shape[:-1], weight.shape[0]), device=x.device, dtype=output_dtype)


_LIB = torch.library.Library("residue", "FRAGMENT")
_LIB.define("mxfp4_linear(Tensor x, Tensor weight, Tensor weight_scale, Tensor indices, Tensor masks, str mode, "
            "ScalarType output_dtype, Tensor? bias=None) -> Tensor")
_LIB.impl("mxfp4_linear", mxfp4_linear, "CUDA")
torch.library.register_fake("residue::mxfp4_linear", _fake_mxfp4_linear, lib=_LIB)
