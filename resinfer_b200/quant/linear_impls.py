"""Linear implementations registered in ``LinearRegistry`` under the reference's names.

The reference registers ``ResidueLinear``, ``ResidueSwapLinear`` and ``NVFP4Linear``
(quant/modelopt_integration/linear_impls.py:30-118) as wrappers around ModelOpt's fake-quantised
modules; here the same names build inference modules that hold packed FP4 weights and run the
``residue::nvfp4_linear`` / ``residue::mxfp4_linear`` ops.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import weight_prep
from .linear_registry import LinearRegistry


def _input_global_scale(linear: nn.Module, kwargs) -> float:
    """amax/(6*448) of the layer's activations; a calibrated ``input_amax`` keyword, else 1.0 amax."""
    amax = float(kwargs.get("input_amax", 1.0))
    return amax / (6.0 * 448.0)


class _Fp4LinearBase(nn.Module):
    """Packed NVFP4 linear: y = nvfp4_linear(x) (+ bias)."""

    ratio: float = 0.0

    def __init__(self, prep: dict, input_global_scale: float, mask: torch.Tensor | None, bias, out_features: int,
                 is_mext_r1: bool):
        super().__init__()
        dev = prep["weight"].device
        for name in ("weight", "weight_scale", "weight_scale_base"):
            self.register_buffer(name, prep[name])
        self.register_buffer("input_global_scale_inv", torch.tensor([1.0 / input_global_scale], dtype=torch.float32, device=dev))
        self.register_buffer("alpha", (prep["weight_global_scale"].to(dev) * input_global_scale).float())
        self.register_buffer("channel_mask", mask if mask is not None else torch.zeros(1, dtype=torch.uint8, device=dev))
        self.bias = bias
        self.k_base, self.num_salient = prep["k_base"], prep["num_salient"]
        self.out_features, self.is_mext_r1 = out_features, is_mext_r1

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .vllm_integration import residue_linear_op  # noqa: F401  (registers the op)
        x2 = x.reshape(-1, x.shape[-1])
        y = torch.ops.residue.nvfp4_linear(
            x2, self.weight, self.input_global_scale_inv, self.weight_scale, self.weight_scale_base,
            self.channel_mask, self.alpha, self.k_base, self.num_salient, 0, self.out_features,
            True, False, self.is_mext_r1)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*x.shape[:-1], self.out_features)

    @classmethod
    def _build(cls, linear: nn.Module, salient_indices, is_mext_r1: bool, kwargs):
        w = linear.weight.data
        prep = weight_prep.quantize_weight_nvfp4(w, None if is_mext_r1 else salient_indices)
        mask = None
        if salient_indices is not None and not is_mext_r1:
            from ..nvfp4.quant import indices_to_channel_masks
            mask = indices_to_channel_masks(salient_indices.to(w.device), w.shape[1])
        return cls(prep, _input_global_scale(linear, kwargs), mask, getattr(linear, "bias", None), w.shape[0],
                   is_mext_r1)


@LinearRegistry.register("NVFP4Linear")
class NVFP4Linear(_Fp4LinearBase):
    """Plain W4A4 NVFP4 linear (no residue)."""

    @classmethod
    def from_linear(cls, linear: nn.Module, **kwargs) -> nn.Module:
        return cls._build(linear, None, False, kwargs)


@LinearRegistry.register("ResidueLinear")
class ResidueLinear(_Fp4LinearBase):
    """NVFP4 linear with residue compensation.  ``ratio`` 1.0 (default) = MEXT on all channels;
    0.125 / 0.25 / 0.5 = KEXT on ``salient_indices`` (or a seeded per-8 selection)."""

    @classmethod
    def from_linear(cls, linear: nn.Module, **kwargs) -> nn.Module:
        ratio = float(kwargs.get("ratio", 1.0))
        if ratio == 1.0:
            return cls._build(linear, None, True, kwargs)
        per8 = {0.125: 1, 0.25: 2, 0.5: 4}.get(ratio)
        if per8 is None:
            raise ValueError(f"Unsupported salient ratio {ratio}")
        idx = kwargs.get("salient_indices")
        if idx is None:
            idx = weight_prep.salient_indices_per8(linear.weight.shape[1], per8, device=linear.weight.device)
        return cls._build(linear, idx, False, kwargs)


@LinearRegistry.register("ResidueSwapLinear")
class ResidueSwapLinear(_Fp4LinearBase):
    """The reference's swapped-residue variant; its kernels are not part of this library."""

    @classmethod
    def from_linear(cls, linear: nn.Module, **kwargs) -> nn.Module:
        raise NotImplementedError("swapped-residue K-extension is not implemented")


__all__ = ["NVFP4Linear", "ResidueLinear", "ResidueSwapLinear"]
