"""FP4 (E2M1), E4M3 and E8M0 codecs, reciprocal providers and the 128x4 scale swizzle.

Test infrastructure (see the package docstring).  All arithmetic is numpy float32 with the
rounding steps written out, so that it can follow the device code operation by operation.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "E2M1_MAGNITUDES", "e2m1_encode", "e2m1_decode", "pack_nibbles", "unpack_nibbles",
    "e4m3_encode", "e4m3_decode", "e8m0_ceil_encode", "e8m0_decode",
    "ExactRcp", "TableRcp", "RecordingRcp", "fma_f32", "bf16_round", "to_bf16_bits",
    "from_bf16_bits", "sf_offset", "sf_buffer_size", "swizzle_scales", "unswizzle_scales",
]

f32 = np.float32

# magnitude of E2M1 code 0..7 (sign is bit 3)   [nvfp4_utils.cuh:143-161 uses cvt.rn.satfinite.e2m1x2.f32]
E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=f32)


def e2m1_encode(v: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit E2M1 code (uint8 0..15), round-to-nearest-even, saturating at 6.

    Ties go to the code with an even mantissa bit: 0.25->0, 0.75->1, 1.25->1, 1.75->2,
    2.5->2, 3.5->4, 5->4.  The sign bit follows the sign of the input, also for results
    that round to zero.
    """
    v = np.asarray(v, dtype=f32)
    a = np.abs(v)
    code = np.zeros(a.shape, dtype=np.uint8)
    code = np.where(a > f32(0.25), 1, code)
    code = np.where(a >= f32(0.75), 2, code)
    code = np.where(a > f32(1.25), 3, code)
    code = np.where(a >= f32(1.75), 4, code)
    code = np.where(a > f32(2.5), 5, code)
    code = np.where(a >= f32(3.5), 6, code)
    code = np.where(a > f32(5.0), 7, code)
    code = np.where(np.isnan(a), 7, code)
    sign = np.signbit(v).astype(np.uint8) << 3
    return (code | sign).astype(np.uint8)


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    """4-bit code -> float32 (exact; mirrors cvt.rn.f16x2.e2m1x2, nvfp4_utils.cuh:185-238)."""
    code = np.asarray(code, dtype=np.uint8)
    mag = E2M1_MAGNITUDES[code & 7]
    return np.where(code & 8, -mag, mag).astype(f32)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[..., K] codes -> [..., K/2] bytes, element 2i in the LOW nibble of byte i."""
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def e4m3_encode(v: np.ndarray):
    """non-negative float32 -> (E4M3 byte, its float32 value); RN-even, saturate at 448.

    Mirrors ``__nv_fp8_e4m3(float)`` as used by encode_sf_to_fp8 (nvfp4_utils.cuh:408-423).
    """
    v = np.asarray(v, dtype=f32)
    nan = np.isnan(v)
    a = np.minimum(np.abs(np.where(nan, 0, v)), f32(448.0)).astype(np.float64)
    # exponent of the quantisation step: normals 2^(e-3), e in [-6, 8]; subnormals step 2^-9
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = np.exp2(e - 3)
    q = np.rint(a / step) * step          # np.rint is round-half-even; a/step is exact
    q = np.minimum(q, 448.0)
    # encode bits from the value
    with np.errstate(divide="ignore"):
        qe = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    normal = q >= 2.0 ** -6
    exp_field = np.where(normal, qe + 7, 0).astype(np.int64)
    man = np.where(normal, np.rint((q / np.exp2(qe) - 1.0) * 8), np.rint(q / 2.0 ** -9)).astype(np.int64)
    byte = ((exp_field << 3) | man).astype(np.uint8)
    sign = (np.signbit(v) & ~nan).astype(np.uint8) << 7
    byte = np.where(nan, np.uint8(0x7F), byte | sign)
    val = np.where(nan, np.nan, np.where(np.signbit(v), -q, q)).astype(f32)
    return byte.astype(np.uint8), val


def e4m3_decode(byte: np.ndarray) -> np.ndarray:
    byte = np.asarray(byte, dtype=np.uint8)
    s = (byte >> 7) & 1
    e = ((byte >> 3) & 0xF).astype(np.int64)
    m = (byte & 7).astype(np.float64)
    val = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(e - 7.0))
    val = np.where((byte & 0x7F) == 0x7F, np.nan, val)
    return np.where(s == 1, -val, val).astype(f32)


def e8m0_ceil_encode(v: np.ndarray) -> np.ndarray:
    """non-negative float32 -> E8M0 byte = smallest power of two >= v (round toward +inf),
    saturating to 0xFE.  Mirrors __nv_cvt_float_to_e8m0(v, __NV_SATFINITE, cudaRoundPosInf)
    (mxfp4_residue_quant.cu:19-29).  v == 0 (or below 2^-127) gives code 0."""
    v = np.asarray(v, dtype=f32)
    bits = v.view(np.uint32) if v.flags["C_CONTIGUOUS"] else np.ascontiguousarray(v).view(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int64)
    man = (bits & 0x7FFFFF).astype(np.int64)
    code = np.where(man != 0, exp + 1, exp)
    code = np.where(exp == 0, np.where(man != 0, 1, 0), code)   # float subnormals round up to 2^-126
    code = np.where(exp == 0xFF, 0xFE, code)                    # inf / nan saturate
    code = np.clip(code, 0, 0xFE)
    return code.astype(np.uint8)


def e8m0_decode(byte: np.ndarray) -> np.ndarray:
    byte = np.asarray(byte, dtype=np.uint8).astype(np.int64)
    return np.exp2(byte - 127.0).astype(f32)


# ------------------------------------------------------------------------------------------
# reciprocal providers: the device code takes rcp.approx.ftz.f32 (nvfp4_utils.cuh:395-399)
# ------------------------------------------------------------------------------------------
class ExactRcp:
    """Correctly rounded float32 reciprocal.  Differs from rcp.approx.ftz.f32 by at most one
    unit in the last place, which can flip a code only on an exact rounding tie."""

    def __call__(self, x):
        x = np.asarray(x, dtype=f32)
        with np.errstate(divide="ignore"):
            return (f32(1.0) / x).astype(f32)


class TableRcp:
    """Reciprocal looked up in a table {float32 bit pattern -> result bit pattern} recorded on
    the device; inputs that are not in the table fall back to the exact reciprocal (counted
    in ``misses``)."""

    def __init__(self, keys: np.ndarray, values: np.ndarray):
        order = np.argsort(keys)
        self.keys = np.asarray(keys, dtype=np.uint32)[order]
        self.values = np.asarray(values, dtype=np.uint32)[order]
        self.misses = 0

    def __call__(self, x):
        x = np.ascontiguousarray(np.asarray(x, dtype=f32))
        bits = x.view(np.uint32).ravel()
        if self.keys.size == 0:
            self.misses += bits.size
            return ExactRcp()(x)
        idx = np.clip(np.searchsorted(self.keys, bits), 0, self.keys.size - 1)
        hit = self.keys[idx] == bits
        exact = ExactRcp()(x).view(np.uint32).ravel()
        out = np.where(hit, self.values[idx], exact).astype(np.uint32)
        self.misses += int((~hit).sum())
        return out.view(f32).reshape(x.shape)


class RecordingRcp:
    """Wraps a device reciprocal ``fn(float32 array) -> float32 array`` and records every
    (input, output) pair so that the pairs can be stored next to a golden fixture."""

    def __init__(self, fn):
        self.fn = fn
        self._k = []
        self._v = []

    def __call__(self, x):
        x = np.ascontiguousarray(np.asarray(x, dtype=f32))
        uniq, inv = np.unique(x.view(np.uint32).ravel(), return_inverse=True)
        res = np.asarray(self.fn(uniq.view(f32)), dtype=f32)
        self._k.append(uniq)
        self._v.append(res.view(np.uint32))
        return res[inv].reshape(x.shape)

    def table(self):
        if not self._k:
            return np.zeros(0, np.uint32), np.zeros(0, np.uint32)
        k = np.concatenate(self._k)
        v = np.concatenate(self._v)
        k, i = np.unique(k, return_index=True)
        return k, v[i]


def fma_f32(a, b, c):
    """round_f32(a*b + c) with a single rounding (a*b is exact in float64)."""
    return (np.asarray(a, np.float64) * np.asarray(b, np.float64) + np.asarray(c, np.float64)).astype(f32)


# ------------------------------------------------------------------------------------------
# bfloat16 helpers (numpy has no bf16: keep bit patterns in uint16)
# ------------------------------------------------------------------------------------------
def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit pattern, round-to-nearest-even."""
    b = np.ascontiguousarray(np.asarray(x, dtype=f32)).view(np.uint32)
    rnd = ((b >> 16) & 1) + np.uint32(0x7FFF)
    return ((b + rnd) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(f32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return from_bf16_bits(to_bf16_bits(x))


# ------------------------------------------------------------------------------------------
# 128x4 swizzled scale-factor layout      [nvfp4_utils.cuh:1080-1107]
# ------------------------------------------------------------------------------------------
def sf_offset(m, kg, k_total: int, vec: int = 16):
    """Byte offset of the scale of row ``m``, k-group ``kg`` in the swizzled buffer of a
    tensor with ``k_total`` columns and ``vec`` elements per scale."""
    m = np.asarray(m, dtype=np.int64)
    kg = np.asarray(kg, dtype=np.int64)
    k_tiles = (k_total + 4 * vec - 1) // (4 * vec)
    return ((m // 128) * (k_tiles * 512) + (kg // 4) * 512 + (m % 32) * 16
            + ((m % 128) // 32) * 4 + (kg % 4))


def sf_buffer_size(rows: int, k_total: int, vec: int = 16) -> int:
    return ((rows + 127) // 128) * ((k_total + 4 * vec - 1) // (4 * vec)) * 512


def swizzle_scales(linear: np.ndarray, vec: int = 16, fill: int = 0) -> np.ndarray:
    """[rows, groups] uint8 -> flat swizzled buffer (padding bytes = ``fill``);
    same result as the reference's swizzle_scales (csrc/nvfp4/scale_layout.py:8-33)."""
    linear = np.asarray(linear, dtype=np.uint8)
    rows, groups = linear.shape
    out = np.full(sf_buffer_size(rows, groups * vec, vec), fill, dtype=np.uint8)
    m, kg = np.meshgrid(np.arange(rows), np.arange(groups), indexing="ij")
    out[sf_offset(m, kg, groups * vec, vec)] = linear
    return out


def unswizzle_scales(buf: np.ndarray, rows: int, groups: int, vec: int = 16,
                     k_total: int | None = None) -> np.ndarray:
    buf = np.asarray(buf, dtype=np.uint8).ravel()
    m, kg = np.meshgrid(np.arange(rows), np.arange(groups), indexing="ij")
    return buf[sf_offset(m, kg, k_total if k_total is not None else groups * vec, vec)]
