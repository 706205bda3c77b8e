"""Host entry points of the block-scaled FP4 Fold GEMM.

Same call signatures as the reference's csrc/common/fold/sm10x/host.py:190-334.  The reference
compiles one CuTeDSL kernel per (tile, cluster, store mode, ...) tactic; here every call goes to the
one tcgen05 kernel of this library, so the tactic arguments are accepted for compatibility and do not
change the result.
"""
from __future__ import annotations

import torch

from ... import ops

DEFAULT_MMA_TILER_MN = (128, 128)
DEFAULT_CLUSTER_SHAPE_MN = (1, 1)
SF_VEC_SIZE = 16


def mext_fold_gemm(weight_fp4: torch.Tensor, act_fp4_rowpair: torch.Tensor, weight_sf: torch.Tensor,
                   act_sf: torch.Tensor, alpha: torch.Tensor | None, out_dtype: torch.dtype = torch.bfloat16,
                   mma_tiler_mn=DEFAULT_MMA_TILER_MN, cluster_shape_mn=DEFAULT_CLUSTER_SHAPE_MN,
                   store_mode: str = "tma", kernel_arch: str = "sm100", ab_stage_override=None,
                   pi_via_layout: bool = False, alpha_res: torch.Tensor | None = None,
                   fp4_format: str = "nvfp4") -> torch.Tensor:
    """Compute GEMM with full-channel residue compensation.

    ``act_fp4_rowpair`` [2M, K/2] holds base / residue codes of token i in rows 2i / 2i+1; the result is
    ``alpha * (base + residue) . W^T`` (``alpha_res`` or a 2-element ``alpha`` scales the residue term
    separately), [M, N] in ``out_dtype``."""
    del mma_tiler_mn, cluster_shape_mn, ab_stage_override, pi_via_layout
    if kernel_arch != "sm100":
        raise ValueError("Fold supports SM100; SM103 Fold is not supported")
    if fp4_format not in ("nvfp4", "mxfp4"):
        raise ValueError(f"unknown FP4 format: {fp4_format}")
    if store_mode not in ("tma", "tma_mext", "direct_mext"):
        raise ValueError(f"unknown store_mode {store_mode!r}")
    n_w, k_packed = weight_fp4.shape
    m2 = act_fp4_rowpair.shape[0]
    assert m2 % 2 == 0, "activation must be row-pair interleaved (even rows)"
    if weight_fp4.stride(0) != k_packed:
        assert weight_fp4.stride(1) == 1, (
            f"weight must stay K-contiguous within a row; got stride {weight_fp4.stride()}")
        assert weight_fp4.stride(0) > k_packed, (
            f"weight row stride {weight_fp4.stride(0)} < width {k_packed}: rows would overlap")
        assert weight_fp4.stride(0) % 32 == 0, (
            f"strided weight row stride {weight_fp4.stride(0)} is not 32B-aligned; "
            "materialise a contiguous base-K prefix for this layer")
    if act_fp4_rowpair.stride(0) != k_packed or act_fp4_rowpair.stride(1) != 1:
        raise ValueError(f"activation must be compact [{m2}, {k_packed}]; got stride {act_fp4_rowpair.stride()}")
    if fp4_format == "mxfp4":
        if alpha_res is not None:
            raise ValueError("MXFP4 has no global residue scale")
        alpha_t = None
    elif alpha_res is not None:
        alpha_t = torch.cat([alpha.reshape(1), alpha_res.reshape(1)]).to(torch.float32)
    else:
        alpha_t = alpha.reshape(-1).to(torch.float32)
    return ops.fp4_gemm(act_fp4_rowpair, act_sf, weight_fp4, weight_sf, alpha_t, m=m2 // 2, fmt=fp4_format,
                        layout="row_pair", out_dtype=out_dtype)


def kext_kloop_gemm_sm100(weight_fp4: torch.Tensor, act_fp4_kext: torch.Tensor, weight_sf: torch.Tensor,
                          act_sf: torch.Tensor, alpha: torch.Tensor, out_dtype=None,
                          mma_tiler_mn=DEFAULT_MMA_TILER_MN, cluster_shape_mn=DEFAULT_CLUSTER_SHAPE_MN) -> torch.Tensor:
    """Compute base and residue GEMM from the K-concatenated activation ([M, K] bytes = 2K codes)."""
    del mma_tiler_mn, cluster_shape_mn
    out_dtype = out_dtype or torch.bfloat16
    n_w, k_packed = weight_fp4.shape
    k = k_packed * 2
    assert weight_fp4.stride(0) == k_packed and weight_fp4.stride(1) == 1, (
        "kloop_tma expects a contiguous weight (mext_r1 weights are)")
    assert act_fp4_kext.shape[1] == k, (
        f"activation must be [rows, {k}] bytes (2K elements), got {tuple(act_fp4_kext.shape)}")
    return ops.fp4_gemm(act_fp4_kext, act_sf, weight_fp4, weight_sf, alpha.reshape(1).to(torch.float32),
                        m=act_fp4_kext.shape[0], fmt="nvfp4", layout="concat_k", out_dtype=out_dtype)
