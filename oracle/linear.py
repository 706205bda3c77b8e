"""Linear-layer oracles: the FP32 product of dequantised operands (GEMM checker) and the
reference's torch-eager quantise / dequantise / matmul path (timed CPU baseline).

Test infrastructure (see the package docstring).

``eager_residue_linear`` restates ResidueQuantLinear._forward_residue_qdq
(quant/modelopt_integration/residue_linear.py:53-136): qdq(x); residue of the selected channels;
qdq(residue); concatenate; extend W with copies of the selected columns; qdq(W'); F.linear.  The
block quantise/dequantise arithmetic of that path lives in NVIDIA ModelOpt (un-vendored, version
not pinned by the reference; util.py:55-56 mentions 0.45), so it is restated here from the
published NVFP4 / MXFP4 recipes with exact divisions: parity of this path is UNPINNED.
"""
from __future__ import annotations

import numpy as np

from .fp4_codec import bf16_round, unswizzle_scales
from .mxfp4_quant import mxfp4_dequant
from .nvfp4_quant import nvfp4_dequant

__all__ = ["dequant_operand", "fp4_linear_reference", "eager_qdq_nvfp4", "eager_qdq_mxfp4",
           "eager_residue_linear", "make_activation", "make_weight"]

f32 = np.float32


def dequant_operand(codes: np.ndarray, sf_swizzled: np.ndarray, fmt: str, k_total: int | None = None):
    """codes [R, K/2] + swizzled scale buffer -> float32 [R, K] (no global scale)."""
    rows, kp = codes.shape
    k = kp * 2
    vec = 16 if fmt == "nvfp4" else 32
    lin = unswizzle_scales(sf_swizzled, rows, k // vec, vec, k_total or k)
    return nvfp4_dequant(codes, lin) if fmt == "nvfp4" else mxfp4_dequant(codes, lin)


def fp4_linear_reference(a_deq: np.ndarray, w_deq: np.ndarray, alpha: float = 1.0,
                         round_bf16: bool = True) -> np.ndarray:
    """y = alpha * a_deq @ w_deq.T accumulated in float64, then float32 (and bf16)."""
    y = (np.asarray(a_deq, np.float64) @ np.asarray(w_deq, np.float64).T) * float(alpha)
    y = y.astype(f32)
    return bf16_round(y) if round_bf16 else y


# ------------------------------------------------------------------------------------------
# torch-eager path (CPU baseline).  torch is imported lazily so the numpy oracle stays light.
# ------------------------------------------------------------------------------------------
_E2M1_BOUNDS = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
_E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def _e2m1_qdq_torch(v):
    import torch
    a = v.abs()
    bounds = torch.tensor(_E2M1_BOUNDS, dtype=v.dtype)
    vals = torch.tensor(_E2M1_VALUES, dtype=v.dtype)
    idx = torch.bucketize(a, bounds)                      # a <= bound -> lower bucket
    # ties: 0.25->0, 0.75->1(up), 1.25->1(down), 1.75->2(up), 2.5->2(down), 3.5->4(up), 5->4(down)
    up_ties = torch.tensor([0.75, 1.75, 3.5], dtype=v.dtype)
    idx = idx + torch.isin(a, up_ties).to(idx.dtype)
    return torch.sign(v) * vals[idx.clamp(max=7)]


def eager_qdq_nvfp4(x, global_amax=None):
    """Fake-quantise x [..., K] to NVFP4 and back (float32).  Global scale amax/(6*448); block
    scale e4m3(block_amax / 6 / gs); values rounded to the E2M1 grid."""
    import torch
    x = x.float()
    amax = x.abs().max() if global_amax is None else torch.as_tensor(global_amax).float()
    gs = (amax / (6.0 * 448.0)).clamp_min(1e-30)
    xb = x.reshape(*x.shape[:-1], -1, 16)
    bmax = xb.abs().amax(dim=-1, keepdim=True)
    sf = (bmax / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn).float()
    denom = sf * gs
    q = _e2m1_qdq_torch(torch.where(denom > 0, xb / denom, torch.zeros_like(xb)))
    return (q * denom).reshape(x.shape)


def eager_qdq_mxfp4(x):
    """Fake-quantise x [..., K] to MXFP4 (32-blocks, power-of-two scale = ceil) and back."""
    import torch
    x = x.float()
    xb = x.reshape(*x.shape[:-1], -1, 32)
    bmax = xb.abs().amax(dim=-1, keepdim=True)
    e = torch.ceil(torch.log2(torch.where(bmax > 0, bmax / 6.0, torch.ones_like(bmax))))
    scale = torch.exp2(e.clamp(-127, 127))
    q = _e2m1_qdq_torch(torch.where(bmax > 0, xb / scale, torch.zeros_like(xb)))
    return (q * scale).reshape(x.shape)


def eager_residue_linear(x, w, salient_indices=None, fmt: str = "nvfp4", out_dtype=None):
    """The torch-eager residue linear on CPU tensors.  ``salient_indices`` None = all channels
    (ratio 1.0 = MEXT).  x [M, K] and w [N, K] in bf16/fp32; returns [M, N] in ``out_dtype``."""
    import torch
    import torch.nn.functional as F
    qdq = eager_qdq_nvfp4 if fmt == "nvfp4" else eager_qdq_mxfp4
    xf = x.float()
    if salient_indices is None:
        salient_indices = torch.arange(x.shape[-1])
    sel = salient_indices.long()
    base = qdq(xf)
    res = xf.index_select(-1, sel) - base.index_select(-1, sel)
    res_q = qdq(res)
    a = torch.cat([base, res_q], dim=-1)
    w_ext = torch.cat([w.float(), w.float().index_select(-1, sel)], dim=-1)
    w_q = qdq(w_ext)
    y = F.linear(a, w_q)
    return y.to(out_dtype or x.dtype)


# ------------------------------------------------------------------------------------------
# seeded synthetic tensors of the benchmark configurations
# ------------------------------------------------------------------------------------------
def make_activation(m: int, k: int, seed: int = 0, outlier_frac: float = 0.01,
                    outlier_gain: float = 20.0) -> np.ndarray:
    """x ~ N(0,1) with ``outlier_frac`` of the channels scaled by ``outlier_gain``; bf16-exact
    float32 [M, K]."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=f32)
    n_out = int(np.ceil(outlier_frac * k))
    ch = np.random.default_rng(seed + 1000).permutation(k)[:n_out]
    x[:, ch] *= f32(outlier_gain)
    return bf16_round(x)


def make_weight(n: int, k: int, seed: int = 1, std: float = 0.02) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return bf16_round(rng.standard_normal((n, k), dtype=f32) * f32(std))
