"""NVFP4 (E2M1 codes, 16-element blocks, E4M3 block scale, FP32 global scale) quantisers.

Test infrastructure (see the package docstring).  Every function takes ``x`` as float32 holding
values that are exactly representable in the input dtype (bf16 / fp16) and ``gs_inv`` as the
reciprocal global scale the device kernels receive (``input_global_scale_inv``,
quant/vllm_integration/linear_method_v2.py:464-479).
"""
from __future__ import annotations

import numpy as np

from .fp4_codec import (ExactRcp, e2m1_decode, e2m1_encode, e4m3_decode, e4m3_encode, fma_f32,
                        pack_nibbles, sf_buffer_size, sf_offset, unpack_nibbles)

__all__ = [
    "LAYOUT_CONCAT", "LAYOUT_ROW_PAIR", "LAYOUT_TILE8", "LAYOUT_CONCAT_K", "LAYOUT_ATTN_TILE8",
    "nvfp4_base_blocks", "nvfp4_mext_blocks", "mext_rows", "nvfp4_quant_mext", "nvfp4_quant_kext",
    "nvfp4_quant_grouped_q", "nvfp4_quant_plain", "nvfp4_dequant", "make_kext_mask",
    "mask_to_indices",
]

f32 = np.float32

# MExtR1LayoutMode, csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:344-353
LAYOUT_CONCAT, LAYOUT_ROW_PAIR, LAYOUT_TILE8, LAYOUT_CONCAT_K, LAYOUT_ATTN_TILE8 = 0, 1, 2, 3, 4


def _mul(a, b):
    return (np.asarray(a, f32) * np.asarray(b, f32)).astype(f32)


def _scale_from_amax(amax, gs, rcp):
    """SF = e4m3(gs * (amax * rcp(6)))  and  mult = gs * rcp(SF) (0 when SF == 0).
    compute_sf_from_max / encode_sf_to_fp8 / compute_output_scale_precise,
    nvfp4_utils.cuh:402-429."""
    rcp6 = rcp(np.array([6.0], dtype=f32))[0]
    sfv = _mul(gs, _mul(amax, rcp6))
    sf_byte, sf_val = e4m3_encode(sfv)
    safe = np.where(sf_val != 0, sf_val, f32(1.0)).astype(f32)
    mult = np.where(sf_val != 0, _mul(gs, rcp(safe)), f32(0.0)).astype(f32)
    return sf_byte, mult


def nvfp4_base_blocks(xb: np.ndarray, gs, rcp=None):
    """xb [..., 16] float32 -> (codes [..., 16], sf_byte [...], mult [...], hat [..., 16])."""
    rcp = rcp or ExactRcp()
    amax = np.abs(xb).max(axis=-1).astype(f32)
    sf_byte, mult = _scale_from_amax(amax, f32(gs), rcp)
    scaled = _mul(xb, mult[..., None])
    codes = e2m1_encode(scaled)
    return codes, sf_byte, mult, e2m1_decode(codes)


def nvfp4_mext_blocks(x: np.ndarray, gs_inv, gs_inv_res=None, rcp=None, fma: bool = True):
    """Base + full residue quantisation of x [M, K] (K % 16 == 0).

    Follows cvt_warp_fp16_to_fp4_mext_r1_fast / _fast16 (nvfp4_utils.cuh:467-556, 614-713):
    residue = x - hat * rcp(mult), which the reference build (--use_fast_math) contracts into one
    fused multiply-add (``fma=True``); ``fma=False`` rounds the product first.
    Returns dict(base_codes [M,K], base_sf [M,K/16], res_codes [M,K], res_sf [M,K/16]).
    """
    rcp = rcp or ExactRcp()
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    assert k % 16 == 0
    gs = f32(gs_inv)
    gs_r = gs if gs_inv_res is None else f32(gs_inv_res)
    xb = x.reshape(m, k // 16, 16)
    codes, sf_byte, mult, hat = nvfp4_base_blocks(xb, gs, rcp)
    safe = np.where(mult != 0, mult, f32(1.0)).astype(f32)
    inv = np.where(mult != 0, rcp(safe), f32(0.0)).astype(f32)
    if fma:
        r = fma_f32(-hat, inv[..., None], xb)
    else:
        r = (xb - _mul(hat, inv[..., None])).astype(f32)
    ramax = np.abs(r).max(axis=-1).astype(f32)
    rsf_byte, rmult = _scale_from_amax(ramax, gs_r, rcp)
    rcodes = e2m1_encode(_mul(r, rmult[..., None]))
    return dict(base_codes=codes.reshape(m, k), base_sf=sf_byte, res_codes=rcodes.reshape(m, k),
                res_sf=rsf_byte, residue=r.reshape(m, k), base_mult=mult)


def mext_rows(i, num_rows: int, layout: int):
    """(base row, residue row, base SF row, residue SF row) of token ``i``.
    compute_mext_r1_{base,residue}[_sf]_row, nvfp4_utils.cuh:1109-1160."""
    i = np.asarray(i, dtype=np.int64)
    if layout in (LAYOUT_TILE8, LAYOUT_ATTN_TILE8):
        base = (i // 8) * 16 + i % 8
        res = base + 8
        if layout == LAYOUT_ATTN_TILE8:
            sfb = (i // 8) * 128 + i % 8
            return base, res, sfb, sfb + 8
        return base, res, base, res
    if layout == LAYOUT_ROW_PAIR:
        return 2 * i, 2 * i + 1, 2 * i, 2 * i + 1
    return i, i + num_rows, i, i + num_rows


def nvfp4_quant_mext(x: np.ndarray, gs_inv, layout: int = LAYOUT_ROW_PAIR, m_pad_multiple=None,
                     gs_inv_res=None, rcp=None, fma: bool = True):
    """Whole-tensor MEXT quantiser in the five output layouts.

    Mirrors scaled_fp4_quant_mext_r1 (csrc/nvfp4/mext.py:97-192) + the kernels at
    csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:113-262.  Returns ``(codes, sf, sf_written)``:
    ``codes`` uint8 [2*M', K/2] (or [M, K] bytes for concat_k), ``sf`` the flat swizzled scale
    buffer and ``sf_written`` a boolean mask of the bytes the reference kernel defines (the
    others are uninitialised memory in the reference, except for attn_tile8 whose buffer is
    zero-filled).
    """
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    if layout in (LAYOUT_TILE8, LAYOUT_ATTN_TILE8):
        # the kernel pads to a multiple of 8 whatever the caller's m_pad_multiple
        # (scaled_fp4_quant_mext_r1_impl, nvfp4_quant_kernels.cu:543-551); a larger caller
        # buffer keeps its extra rows untouched
        out_m = (m + 7) // 8 * 8
    else:
        out_m = m
    xp = np.zeros((out_m, k), dtype=f32)
    xp[:m] = x
    q = nvfp4_mext_blocks(xp, gs_inv, gs_inv_res, rcp, fma)
    base_p, res_p = pack_nibbles(q["base_codes"]), pack_nibbles(q["res_codes"])
    rows = np.arange(out_m)
    kg = np.arange(k // 16)
    if layout == LAYOUT_CONCAT_K:
        codes = np.concatenate([base_p, res_p], axis=1)                      # [M, K] bytes
        size = sf_buffer_size(out_m, 2 * k)
        sf = np.zeros(size, np.uint8)
        written = np.zeros(size, bool)
        ob = sf_offset(rows[:, None], kg[None, :], 2 * k)
        orr = sf_offset(rows[:, None], kg[None, :] + k // 16, 2 * k)
    else:
        br, rr, bsr, rsr = mext_rows(rows, out_m, layout)
        codes = np.zeros((2 * out_m, k // 2), np.uint8)
        codes[br] = base_p
        codes[rr] = res_p
        if layout == LAYOUT_ATTN_TILE8:
            size = (out_m // 8) * ((k + 63) // 64) * 512
        else:
            size = sf_buffer_size(2 * out_m, k)
        sf = np.zeros(size, np.uint8)
        written = np.zeros(size, bool)
        ob = sf_offset(bsr[:, None], kg[None, :], k)
        orr = sf_offset(rsr[:, None], kg[None, :], k)
    sf[ob] = q["base_sf"]
    sf[orr] = q["res_sf"]
    written[ob] = True
    written[orr] = True
    if layout == LAYOUT_ATTN_TILE8:
        written[:] = True
    return codes, sf, written


def make_kext_mask(k: int, per8: int, seed: int = 2) -> np.ndarray:
    """uint8 [K/8]: exactly ``per8`` bits set per byte, chosen uniformly at random (seeded)."""
    rng = np.random.default_rng(seed)
    mask = np.zeros(k // 8, dtype=np.uint8)
    for g in range(k // 8):
        for b in rng.choice(8, size=per8, replace=False):
            mask[g] |= np.uint8(1 << int(b))
    return mask


def mask_to_indices(mask: np.ndarray) -> np.ndarray:
    """Selected channels in increasing order (bit b of mask[g] = channel 8g+b)."""
    bits = np.unpackbits(np.asarray(mask, np.uint8)[:, None], axis=1, bitorder="little")
    return np.flatnonzero(bits.ravel()).astype(np.int64)


def nvfp4_quant_kext(x: np.ndarray, gs_inv, mask: np.ndarray, per8: int, rcp=None, fma: bool = True):
    """KEXT: base codes for all K channels, then the residues of the masked channels.

    Mirrors cvt_warp_fp16_to_fp4 (nvfp4_utils.cuh:895-1019), the pack8 kernels
    (csrc/nvfp4/cuda/nvfp4_residue_pack8.cu:102-304) and the offsets at nvfp4_utils.cuh:1022-1045,
    1185-1217: residue j (selected channels in increasing order) is logical column K+j; one
    scale per 16 consecutive residues, same global scale as the base.  Rows up to the next
    multiple of 128 get scale 0.  Returns ``(codes [M,(K+S)/2], sf, sf_written)``.
    """
    rcp = rcp or ExactRcp()
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    sel = mask_to_indices(mask)
    s = sel.size
    assert s == k // 8 * per8 and s % 16 == 0 and k % 16 == 0
    gs = f32(gs_inv)
    q = nvfp4_mext_blocks(x, gs, None, rcp, fma)            # residue field = x - deq(q(x))
    r = q["residue"][:, sel].reshape(m, s // 16, 16)
    ramax = np.abs(r).max(axis=-1).astype(f32)
    rsf, rmult = _scale_from_amax(ramax, gs, rcp)
    rcodes = e2m1_encode(_mul(r, rmult[..., None])).reshape(m, s)
    codes = np.concatenate([pack_nibbles(q["base_codes"]), pack_nibbles(rcodes)], axis=1)
    n_ext = k + s
    rows_eff = (m + 127) // 128 * 128
    size = sf_buffer_size(m, n_ext)
    sf = np.zeros(size, np.uint8)
    written = np.zeros(size, bool)
    all_rows = np.arange(rows_eff)[:, None]
    ob = sf_offset(all_rows, np.arange(k // 16)[None, :], n_ext)
    orr = sf_offset(all_rows, (k // 16 + np.arange(s // 16))[None, :], n_ext)
    written[ob] = True
    written[orr] = True
    sf[ob[:m]] = q["base_sf"]
    sf[orr[:m]] = rsf
    return codes, sf, written


def nvfp4_quant_plain(x: np.ndarray, gs_inv, rcp=None):
    """Plain NVFP4 quantisation (no residue): codes [M, K/2] and the swizzled scale buffer
    (padding rows / k-groups zero).  Used by the harness for offline weight quantisation."""
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    codes, sf_byte, _, _ = nvfp4_base_blocks(x.reshape(m, k // 16, 16), f32(gs_inv), rcp or ExactRcp())
    sf = np.zeros(sf_buffer_size(m, k), np.uint8)
    sf[sf_offset(np.arange(m)[:, None], np.arange(k // 16)[None, :], k)] = sf_byte
    return pack_nibbles(codes.reshape(m, k)), sf


def nvfp4_quant_grouped_q(q: np.ndarray, rcp=None, fma: bool = True):
    """ResAttn query quantiser: q [B, Hkv, G, D] -> (q_pack [B,Hkv,P,D/2], q_sf flat).

    Rows 0..G-1 hold the base codes, rows P/2..P/2+G-1 the residue codes (P = 8 for G == 4, else
    16), other rows stay zero; global scale 1.0; each (b, hkv) owns a private 128-row swizzled
    scale tile.  Mirrors quantize_mext_grouped_q_kernel,
    csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:616-689."""
    q = np.asarray(q, dtype=f32)
    b, h, g, d = q.shape
    p = 8 if g == 4 else 16
    res = nvfp4_mext_blocks(q.reshape(b * h * g, d), f32(1.0), None, rcp, fma)
    pack = np.zeros((b, h, p, d // 2), np.uint8)
    pack[:, :, :g] = pack_nibbles(res["base_codes"]).reshape(b, h, g, d // 2)
    pack[:, :, p // 2:p // 2 + g] = pack_nibbles(res["res_codes"]).reshape(b, h, g, d // 2)
    groups = d // 16
    sf = np.zeros((b * h, 128 * groups), np.uint8)
    rows = np.arange(g)[:, None]
    kg = np.arange(groups)[None, :]
    sf[:, sf_offset(rows, kg, d)] = res["base_sf"].reshape(b * h, g, groups)
    sf[:, sf_offset(rows + p // 2, kg, d)] = res["res_sf"].reshape(b * h, g, groups)
    return pack, sf.ravel()


def nvfp4_dequant(packed: np.ndarray, sf_linear: np.ndarray, global_scale=1.0) -> np.ndarray:
    """codes [R, K/2] + linear E4M3 scale bytes [R, K/16] -> float32 [R, K] * global_scale."""
    vals = e2m1_decode(unpack_nibbles(packed))
    r, k = vals.shape
    sfv = e4m3_decode(sf_linear).astype(f32)
    out = vals.reshape(r, k // 16, 16) * sfv[:, :, None]
    return (out.reshape(r, k) * f32(global_scale)).astype(f32)
