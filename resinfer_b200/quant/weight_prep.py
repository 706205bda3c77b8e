"""Offline weight preparation: FP4 quantisation, K extension and scale swizzling in plain torch.

The reference prepares weights offline with NVIDIA ModelOpt and loads them from a checkpoint
(quant/modelopt_integration/residue_linear.py:75-91 extends W with copies of the salient columns;
quant/vllm_integration/linear_method_v2.py:464-479 derives ``alpha`` and the reciprocal activation
scale).  This module produces tensors with the same contract from a dense weight, so that layers and
benchmarks can be built without a checkpoint:

    NVFP4: weight uint8 [N, Kx/2], weight_scale = 128x4-swizzled E4M3 bytes over Kx,
           weight_scale_base = the same over the base K prefix, weight_global_scale (FP32)
    MXFP4: weight uint8 [N, Kp/2], weight_scale = 128x4-swizzled E8M0 bytes over Kp

Runs on the tensor's device (CPU or CUDA); it is preparation code, not a hot path.
"""
from __future__ import annotations

import torch

_E2M1_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_E2M1_UP_TIES = (0.75, 1.75, 3.5)          # ties that round to the larger code (even mantissa)


def e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    """float -> uint8 E2M1 codes (sign in bit 3), round-to-nearest-even, saturating at 6."""
    a = v.abs().float()
    idx = torch.bucketize(a, torch.tensor(_E2M1_BOUNDS, device=v.device))
    idx = idx + torch.isin(a, torch.tensor(_E2M1_UP_TIES, device=v.device)).to(idx.dtype)
    idx = idx.clamp(max=7)
    return (idx | (torch.signbit(v).to(idx.dtype) << 3)).to(torch.uint8)


def pack_codes(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] codes -> [..., K/2] bytes, even element in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def swizzle_scales_any(scales: torch.Tensor) -> torch.Tensor:
    """uint8 [M, G] -> flat 128x4-swizzled buffer (zero padded); works on any device."""
    rows, groups = scales.shape
    rt, kt = (rows + 127) // 128, (groups + 3) // 4
    pad = torch.zeros((rt * 128, kt * 4), dtype=torch.uint8, device=scales.device)
    pad[:rows, :groups] = scales
    return pad.reshape(rt, 4, 32, kt, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(-1)


def extend_weight(w: torch.Tensor, salient_indices: torch.Tensor | None) -> torch.Tensor:
    """[W | W[:, sel]] -- the K extension that pairs with the KEXT activation layout."""
    if salient_indices is None or salient_indices.numel() == 0:
        return w
    return torch.cat([w, w.index_select(-1, salient_indices.to(w.device).long())], dim=-1)


def _nvfp4_blocks(w: torch.Tensor, gs: torch.Tensor):
    n, k = w.shape
    wb = w.float().reshape(n, k // 16, 16)
    amax = wb.abs().amax(dim=-1)
    sf = (amax / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn)
    sfv = sf.float() * gs
    q = torch.where(sfv[..., None] > 0, wb / sfv[..., None], torch.zeros_like(wb))
    return e2m1_codes(q).reshape(n, k), sf.view(torch.uint8)


def quantize_weight_nvfp4(w: torch.Tensor, salient_indices: torch.Tensor | None = None) -> dict:
    """Dense weight [N, K] -> NVFP4 tensors for ``residue::nvfp4_linear`` (K % 64 == 0)."""
    n, k = w.shape
    gs = (w.float().abs().amax() / (6.0 * 448.0)).clamp_min(1e-30)
    w_ext = extend_weight(w, salient_indices)
    codes, sf = _nvfp4_blocks(w_ext, gs)
    base_sf = sf[:, :k // 16].contiguous()
    return dict(weight=pack_codes(codes), weight_scale=swizzle_scales_any(sf),
                weight_scale_base=swizzle_scales_any(base_sf), weight_global_scale=gs.reshape(1).float(),
                weight_scale_raw=sf,                       # E4M3 bytes [N, (K+S)/16] as a checkpoint stores them
                k_base=k, num_salient=0 if salient_indices is None else int(salient_indices.numel()))


def quantize_weight_mxfp4(w: torch.Tensor, salient_indices: torch.Tensor | None = None,
                          k_alignment: int = 128) -> dict:
    """Dense weight [N, K] -> MXFP4 tensors (E8M0 'ceil' scales) for ``residue::mxfp4_linear``."""
    n, k = w.shape
    w_ext = extend_weight(w, salient_indices).float()
    kx = w_ext.shape[1]
    kp = -(-kx // k_alignment) * k_alignment
    if kp != kx:
        w_ext = torch.nn.functional.pad(w_ext, (0, kp - kx))
    wb = w_ext.reshape(n, kp // 32, 32)
    amax = wb.abs().amax(dim=-1)
    mant, exp = torch.frexp(amax / 6.0)                    # amax/6 = mant * 2^exp, mant in [0.5, 1)
    e = torch.where(mant == 0.5, exp - 1, exp) + 127        # smallest power of two >= amax/6
    e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(0, 254)
    scale = torch.exp2(e.float() - 127.0)
    q = torch.where(amax[..., None] > 0, wb / scale[..., None], torch.zeros_like(wb))
    codes = e2m1_codes(q).reshape(n, kp)
    return dict(weight=pack_codes(codes), weight_scale=swizzle_scales_any(e.to(torch.uint8)), k_base=k,
                weight_scale_raw=e.to(torch.uint8),        # E8M0 bytes [N, Kp/32] as a checkpoint stores them
                k_padded=kp, num_salient=0 if salient_indices is None else int(salient_indices.numel()))


def salient_indices_per8(k: int, per8: int, seed: int = 2, device="cpu") -> torch.Tensor:
    """Seeded synthetic selection: ``per8`` channels chosen uniformly in every group of eight
    (sorted int64 indices) -- the mask contract of the KEXT quantisers."""
    g = torch.Generator().manual_seed(seed)
    pick = torch.rand(k // 8, 8, generator=g).argsort(dim=1)[:, :per8].sort(dim=1).values
    return (pick + torch.arange(k // 8)[:, None] * 8).reshape(-1).to(device)
