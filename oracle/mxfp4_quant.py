"""MXFP4 (E2M1 codes, 32-element blocks, E8M0 power-of-two scale, no global scale) quantisers.

Test infrastructure (see the package docstring).  Follows cvt_to_mxfp4_residue
(csrc/mxfp4/cuda/mxfp4_residue_quant.cu:84-265): every multiply / subtract is an explicit
round-to-nearest float32 operation there, so no fused multiply-add appears here; only
``rcp(6)`` is an approximate reciprocal.
"""
from __future__ import annotations

import numpy as np

from .fp4_codec import (ExactRcp, e2m1_decode, e2m1_encode, e8m0_ceil_encode, e8m0_decode,
                        pack_nibbles, sf_buffer_size, sf_offset, unpack_nibbles)
from .nvfp4_quant import LAYOUT_ROW_PAIR, LAYOUT_TILE8, mask_to_indices, mext_rows

__all__ = ["mxfp4_blocks", "mxfp4_quant_mext", "mxfp4_quant_selective", "mxfp4_quant_plain",
           "mxfp4_dequant"]

f32 = np.float32


def _mul(a, b):
    return (np.asarray(a, f32) * np.asarray(b, f32)).astype(f32)


def _pow2(exp_field):
    """float32 with exponent field ``exp_field`` and zero mantissa (0 -> 0.0)."""
    return (np.asarray(exp_field, dtype=np.uint32) << np.uint32(23)).view(f32)


def mxfp4_blocks(xb: np.ndarray, rcp=None):
    """xb [..., 32] -> (codes, e8m0 byte [...], dequantised values [..., 32]).
    compute_mxfp4_scale + quantize_fp32_vec16<true>, mxfp4_residue_quant.cu:19-29, 55-81."""
    rcp = rcp or ExactRcp()
    rcp6 = rcp(np.array([6.0], dtype=f32))[0]
    amax = np.abs(xb).max(axis=-1).astype(f32)
    e = e8m0_ceil_encode(_mul(amax, rcp6))
    mult = np.where(e == 0, f32(0.0), _pow2(254 - e.astype(np.int64)))
    codes = e2m1_encode(_mul(xb, mult[..., None]))
    deq = _mul(e2m1_decode(codes), e8m0_decode(e)[..., None])
    return codes, e, deq


def _store_sf(rows, groups_idx, values, total_rows, k_total, swizzle):
    if swizzle:
        buf = np.zeros(sf_buffer_size(total_rows, k_total, 32), np.uint8)
        buf[sf_offset(rows[:, None], groups_idx[None, :], k_total, 32)] = values
        return buf
    buf = np.zeros((total_rows, k_total // 32), np.uint8)
    buf[rows[:, None], groups_idx[None, :]] = values
    return buf


def mxfp4_quant_mext(x: np.ndarray, swizzle: bool = True, tile8: bool = False,
                     m_pad_multiple=None, rcp=None):
    """MXFP4 MEXT: base and full-residue rows in row_pair (or tile8) layout.

    Returns (codes [rows, K/2], sf) with rows = 2*M (row_pair) or 2*ceil(M/pad)*pad (tile8);
    sf is the flat 128x4-swizzled buffer (``swizzle``) or linear [rows, K/32]; padding scales and
    padded tile8 rows are zero, as the reference kernel writes them
    (mxfp4_residue_quant.cu:117-146)."""
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    assert k % 32 == 0
    if tile8:
        mult = 8 if m_pad_multiple is None else int(m_pad_multiple)
        out_m = (m + mult - 1) // mult * mult
    else:
        out_m = m
    xb = x.reshape(m, k // 32, 32)
    codes, e, deq = mxfp4_blocks(xb, rcp)
    r = (xb - deq).astype(f32)                                   # __fsub_rn
    rcodes, er, _ = mxfp4_blocks(r, rcp)
    layout = LAYOUT_TILE8 if tile8 else LAYOUT_ROW_PAIR
    br, rr, _, _ = mext_rows(np.arange(m), m, layout)
    out = np.zeros((2 * out_m, k // 2), np.uint8)
    out[br] = pack_nibbles(codes.reshape(m, k))
    out[rr] = pack_nibbles(rcodes.reshape(m, k))
    rows = np.concatenate([br, rr])
    vals = np.concatenate([e, er], axis=0)
    sf = _store_sf(rows, np.arange(k // 32), vals, 2 * out_m, k, swizzle)
    return out, sf


def mxfp4_quant_selective(x: np.ndarray, mask: np.ndarray, per8: int, kp: int | None = None,
                          swizzle: bool = True, rcp=None):
    """MXFP4 KEXT: base codes of all K channels, then the residues of the masked channels
    (one scale per 32 consecutive residues), zero padded to ``kp`` columns
    (default ceil((K+S)/128)*128, csrc/mxfp4/selective.py:13-18).
    mxfp4_residue_quant.cu:197-258."""
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    sel = mask_to_indices(mask)
    s = sel.size
    assert s == k // 8 * per8
    if kp is None:
        kp = (k + s + 127) // 128 * 128
    xb = x.reshape(m, k // 32, 32)
    codes, e, deq = mxfp4_blocks(xb, rcp)
    r = (xb - deq).astype(f32).reshape(m, k)[:, sel]
    s_pad = (s + 31) // 32 * 32
    rp = np.zeros((m, s_pad), f32)
    rp[:, :s] = r
    rcodes, er, _ = mxfp4_blocks(rp.reshape(m, s_pad // 32, 32), rcp)
    rcodes = rcodes.reshape(m, s_pad)
    out = np.zeros((m, kp // 2), np.uint8)
    out[:, :k // 2] = pack_nibbles(codes.reshape(m, k))
    n8 = (s + 7) // 8 * 8                                       # the kernel stores whole 8-packs
    out[:, k // 2:k // 2 + n8 // 2] = pack_nibbles(rcodes[:, :n8])
    groups = np.arange(k // 32 + s_pad // 32)
    vals = np.concatenate([e, er], axis=1)
    sf = _store_sf(np.arange(m), groups, vals, m, kp, swizzle)
    return out, sf


def mxfp4_quant_plain(x: np.ndarray, swizzle: bool = True, rcp=None):
    """Plain MXFP4 quantisation with the same 'ceil' scale recipe (harness weight prep)."""
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    codes, e, _ = mxfp4_blocks(x.reshape(m, k // 32, 32), rcp)
    sf = _store_sf(np.arange(m), np.arange(k // 32), e, m, k, swizzle)
    return pack_nibbles(codes.reshape(m, k)), sf


def mxfp4_dequant(packed: np.ndarray, sf_linear: np.ndarray) -> np.ndarray:
    vals = e2m1_decode(unpack_nibbles(packed))
    r, k = vals.shape
    out = vals.reshape(r, k // 32, 32) * e8m0_decode(sf_linear)[:, :, None]
    return out.reshape(r, k).astype(f32)
