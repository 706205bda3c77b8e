"""``residue::nvfp4_linear`` -- the opaque NVFP4 linear op (online quantiser + FP4 GEMM).

Same 14-argument schema, fake implementation and routing rule as the reference's
quant/vllm_integration/residue_linear_op.py:140-194 and
quant/flashinfer_integration/nvfp4_linear_adapter.py:31-41:

    fold (row-pair quantiser + fold GEMM)   fold-eligible layers while M <= 128 (RESIDUE_DECODE_MEXT_MAX_M),
                                            ratio-1 layers up to M <= 512 (RESIDUE_MEXT_FOLD_MAX_M)
    ratio1_prefill (K-concat quantiser)     ratio-1 layers above that
    k_ext (masked residue along K)          selective layers otherwise
    plain                                   layers without salient channels

Every route is two launches of this library (quantiser, then the tcgen05 GEMM, chained with
programmatic dependent launch); there is no autotuner, no second backend and no fallback.
"""
from __future__ import annotations

import torch

from ... import nvfp4, ops
from .env_contract import settings

_LAYOUT_ROW_PAIR = 1
_LAYOUT_CONCAT_K = 3


def fold_max_m_for(arch: str | None) -> int:
    configured = settings().decode_max_m
    return configured if configured is not None else (128 if arch is not None else 64)


def mext_fold_max_m_for(arch: str | None) -> int:
    decode_max = fold_max_m_for(arch)
    if arch is None:
        return decode_max
    configured = settings().ratio1_max_m
    return max(decode_max, configured if configured is not None else 512)


_ARCH_BY_DEVICE: dict = {}


def _sm10x_fold_arch(device=None) -> str | None:
    if settings().disable_sm10x:
        return None
    key = None if device is None else torch.device(device).index
    if key not in _ARCH_BY_DEVICE:                         # the capability of a device does not change
        major, minor = torch.cuda.get_device_capability(device)
        from ...nvfp4.cute_fold.tactics import kernel_arch_for_capability
        _ARCH_BY_DEVICE[key] = kernel_arch_for_capability(major, minor) if major == 10 else None
    return _ARCH_BY_DEVICE[key]


def _quant_mext(x: torch.Tensor, scale_inv: torch.Tensor, layout: int):
    """MEXT quantiser straight through the C ABI (same kernel and bytes as
    ``nvfp4.scaled_fp4_quant_mext_r1``; the hot path skips that wrapper's option parsing and the second
    dispatcher round trip)."""
    from ... import _cabi
    lib = _cabi.load()
    m, k = x.shape
    if k % 16 or x.stride(1) != 1:
        raise ValueError(f"scaled_fp4_quant_mext_r1 requires compact rows with K multiple of 16, got {tuple(x.shape)}")
    dev = x.device
    codes = torch.empty((m, k) if layout == _LAYOUT_CONCAT_K else (2 * m, k // 2), dtype=torch.uint8, device=dev)
    k_groups = ((2 * k if layout == _LAYOUT_CONCAT_K else k) + 63) // 64
    rows = m if layout == _LAYOUT_CONCAT_K else 2 * m
    sf = torch.empty(((rows + 127) // 128) * k_groups * 512, dtype=torch.uint8, device=dev)
    st = lib.ri_nvfp4_quant_mext(x.data_ptr(), _cabi.torch_dtype_code(x.dtype), m, k, x.stride(0),
                                 scale_inv.data_ptr(), scale_inv.numel(), codes.data_ptr(), codes.numel(),
                                 sf.data_ptr(), sf.numel(), layout, 1, _cabi.current_stream(dev))
    _cabi.check(st, "nvfp4::scaled_fp4_quant_mext_r1")
    return codes, sf


def fold_prefers_concat_k(m: int, k: int) -> bool:
    """The fold contraction has two operand layouts with the same arithmetic: base / residue as adjacent rows
    (row_pair: 2 M accumulator columns) or side by side along K (concat_k: M columns, two MMA groups per weight
    tile).  Up to 64 tokens row_pair is faster; above, its 256-column accumulator cannot be double-buffered and
    concat_k wins by 10-20 % (measured on B200 for the four projections of the benchmark model)."""
    return m > 64 and k % 256 == 0


def _route(m: int, *, fold_eligible: bool, ratio1: bool, num_salient: int, arch: str | None,
           fold_max_m: int, ratio1_fold_max_m: int, force_fold: bool) -> str:
    """Which numerical path serves ``m`` tokens (reference: nvfp4_linear_adapter.py:31-41)."""
    fold = fold_eligible and arch == "sm100" and (ratio1 or force_fold or m <= fold_max_m)
    if fold:
        return "ratio1_prefill" if ratio1 and m > ratio1_fold_max_m else "sm10x_fold"
    if ratio1:
        return "invalid_mext"
    return "plain" if num_salient == 0 else "k_ext"


def _base_weight_view(weight: torch.Tensor, k_base: int) -> torch.Tensor:
    packed_k = k_base // 2
    if packed_k > weight.shape[1]:
        raise ValueError("base K exceeds packed weight width")
    return weight if packed_k == weight.shape[1] else weight[:, :packed_k]


def _nvfp4_linear_impl(x, weight, scale_inv, weight_scale, weight_scale_base, mask, alpha, *, k_base,
                       num_salient, padding, output_size, fold_eligible, use_swap, ratio1):
    m, k = x.shape
    cfg = settings()
    arch = _sm10x_fold_arch(x.device)
    route = _route(m, fold_eligible=fold_eligible, ratio1=ratio1, num_salient=num_salient, arch=arch,
                   fold_max_m=fold_max_m_for(arch), ratio1_fold_max_m=mext_fold_max_m_for(arch),
                   force_fold=cfg.force_fold)
    if route == "invalid_mext":
        raise RuntimeError("Ratio-1 residue requires a prepared Fold path")
    if use_swap:
        raise NotImplementedError("swapped-residue layout is not supported")
    if padding:
        # K padding exists for another backend's alignment rule; this GEMM takes K % 64 == 0 as is
        raise NotImplementedError("weights_padding_cols != 0 is not supported")
    if route in ("sm10x_fold", "ratio1_prefill"):
        w_base = _base_weight_view(weight, k_base)
        if route == "sm10x_fold" and not fold_prefers_concat_k(m, k):
            codes, sf = _quant_mext(x, scale_inv, _LAYOUT_ROW_PAIR)
            return ops.fp4_gemm(codes, sf, w_base, weight_scale_base, alpha, m=m, fmt="nvfp4",
                                layout="row_pair", out_dtype=x.dtype)
        codes, sf = _quant_mext(x, scale_inv, _LAYOUT_CONCAT_K)
        return ops.fp4_gemm(codes, sf, w_base, weight_scale_base, alpha.reshape(-1)[:1], m=m, fmt="nvfp4",
                            layout="concat_k", out_dtype=x.dtype)
    if route == "plain":
        codes = torch.empty((m, k // 2), dtype=torch.uint8, device=x.device)
        sf = torch.empty(((m + 127) // 128) * ((k + 63) // 64) * 512, dtype=torch.uint8, device=x.device)
        torch.ops.nvfp4.scaled_fp4_quant_mext_r1(codes, x, sf, scale_inv, 0, 5, True)
    else:
        codes, sf = nvfp4.scaled_fp4_quant_with_mask(x, scale_inv, mask, num_salient, use_swapped_residue=False)
    return ops.fp4_gemm(codes, sf, weight, weight_scale, alpha.reshape(-1)[:1], m=m, fmt="nvfp4", layout="plain",
                        out_dtype=x.dtype)


def nvfp4_linear(x: torch.Tensor, weight: torch.Tensor, input_global_scale_inv: torch.Tensor,
                 weight_scale: torch.Tensor, weight_scale_base: torch.Tensor, channel_mask: torch.Tensor,
                 alpha: torch.Tensor, k_base: int, num_salient: int, weights_padding_cols: int,
                 output_size: int, fold_eligible: bool, use_swap: bool, is_mext_r1: bool) -> torch.Tensor:
    """y[M, N] = NVFP4 linear of x[M, K] with residue compensation (MEXT or KEXT by layer type and M)."""
    if x.shape[0] == 0:
        return x.new_empty((0, output_size if output_size > 0 else weight.shape[0]))
    with ops._on_device(x.device):
        out = _nvfp4_linear_impl(
            x, weight, input_global_scale_inv, weight_scale, weight_scale_base, channel_mask, alpha,
            k_base=int(k_base), num_salient=int(num_salient), padding=int(weights_padding_cols),
            output_size=int(output_size), fold_eligible=bool(fold_eligible), use_swap=bool(use_swap),
            ratio1=bool(is_mext_r1))
    return out[:, :output_size].contiguous() if 0 < output_size < out.shape[1] else out


def _nvfp4_linear_fake(x, weight, input_global_scale_inv, weight_scale, weight_scale_base, channel_mask, alpha,
                       k_base, num_salient, weights_padding_cols, output_size, fold_eligible, use_swap,
                       is_mext_r1):
    n = int(output_size) if int(output_size) > 0 else weight.shape[0]
    return torch.empty(x.shape[0], n, dtype=x.dtype, device=x.device)


# Registered straight on the dispatcher (CUDA key + fake kernel): an opaque op for torch.compile like the
# reference's, without the per-call Python wrapper layers of torch.library.custom_op (about 25 us per call).
_LIB = torch.library.Library("residue", "FRAGMENT")
_LIB.define("nvfp4_linear(Tensor x, Tensor weight, Tensor input_global_scale_inv, Tensor weight_scale, "
            "Tensor weight_scale_base, Tensor channel_mask, Tensor alpha, int k_base, int num_salient, "
            "int weights_padding_cols, int output_size, bool fold_eligible, bool use_swap, bool is_mext_r1) -> Tensor")
_LIB.impl("nvfp4_linear", nvfp4_linear, "CUDA")
torch.library.register_fake("residue::nvfp4_linear", _nvfp4_linear_fake, lib=_LIB)
