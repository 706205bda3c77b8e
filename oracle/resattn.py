"""ResAttn oracle: residue-compensated paged NVFP4-KV decode attention (one query token).

Test infrastructure (see the package docstring).  Restates the semantics of the reference's
decode kernel (csrc/resattn/kernel_paged_decode.py): the query is quantised to NVFP4 plus an
NVFP4 residue (nvfp4_quant_kernels.cu:616-689), both rows are multiplied with the dequantised
keys and the two score rows are summed before the softmax (:1905-1913); positions >= seq_len
are masked (:1888-1900); the score scale is sm_scale * k_global_scale (attn/decode.py:92,158);
the output is O / l * v_global_scale in BF16 (:2193-2203).  The reference additionally rounds P
and the dequantised V to E4M3 before its FP8 PV product (:1958-1963, qmul4.py:45) while it keeps
the row sum in unrounded FP32 (:1965-1969); that approximation is optional here
(``p_e4m3`` / ``v_e4m3``) and off by default, so the default oracle is the exact attention over
the dequantised cache.  The reference kernel itself cannot be built on this toolchain (it needs a
CUDA 13.4 PTX compiler), so attention parity is UNPINNED and stated as a tolerance.
"""
from __future__ import annotations

import numpy as np

from .fp4_codec import (bf16_round, e2m1_decode, e4m3_decode, e4m3_encode, sf_offset,
                        unpack_nibbles)
from .nvfp4_quant import nvfp4_quant_grouped_q, nvfp4_quant_plain

__all__ = ["make_paged_kv", "dequant_paged", "resattn_decode_reference", "merge_splits",
           "dequant_grouped_q", "quantize_attention_output_nvfp4"]

f32 = np.float32


def make_paged_kv(seq_lens, num_kv_heads: int, head_dim: int, page_size: int, seed: int = 3,
                  extra_pages: float = 0.1, scale_range: float = 6.0 * 448.0):
    """Seeded synthetic NVFP4 paged KV cache.

    K, V ~ N(0,1) in BF16, quantised to NVFP4 (16-blocks along head_dim, per-tensor global scale
    amax/scale_range: 6*448 uses the whole E4M3 range for the block scales; 448 is the convention of an
    FP8-range cache, where code x block scale never exceeds 448 -- the range the reference's E4M3
    expansion of V, mul.rn.satfinite.e4m3x4 in csrc/resattn/qmul4.py:45, can hold without saturating).
    Pages of all sequences are a random permutation of the pool.  Returns a dict
    with k_data/v_data uint8 [pages, Hkv, page, D/2], k_sf/v_sf uint8 [pages, Hkv, page, D/16]
    (linear E4M3 bytes), block_tables int32 [B, max_pages] (-1 = unused), seq_lens int32 [B],
    k_global_scale, v_global_scale."""
    rng = np.random.default_rng(seed)
    seq_lens = np.asarray(seq_lens, dtype=np.int32)
    pages_per = (seq_lens + page_size - 1) // page_size
    total = int(pages_per.sum())
    pool = int(np.ceil(total * (1.0 + extra_pages))) + 1
    perm = np.random.default_rng(seed + 1).permutation(pool)[:total].astype(np.int32)
    bt = np.full((seq_lens.size, int(max(1, pages_per.max()))), -1, dtype=np.int32)
    o = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[o:o + n]
        o += n
    out = {}
    for name in ("k", "v"):
        x = bf16_round(rng.standard_normal((pool * num_kv_heads * page_size, head_dim), dtype=f32))
        gs = f32(np.abs(x).max() / scale_range)
        codes, sf_sw = nvfp4_quant_plain(x, f32(1.0) / gs)
        rows = np.arange(x.shape[0])[:, None]
        sf_lin = sf_sw[sf_offset(rows, np.arange(head_dim // 16)[None, :], head_dim)]
        out[f"{name}_data"] = codes.reshape(pool, num_kv_heads, page_size, head_dim // 2)
        out[f"{name}_sf"] = sf_lin.reshape(pool, num_kv_heads, page_size, head_dim // 16)
        out[f"{name}_global_scale"] = float(gs)
    out.update(block_tables=bt, seq_lens=seq_lens, page_size=page_size)
    return out


def dequant_paged(data: np.ndarray, sf: np.ndarray) -> np.ndarray:
    """[pages, H, page, D/2] codes + [pages, H, page, D/16] E4M3 bytes -> float32 [pages,H,page,D]."""
    vals = e2m1_decode(unpack_nibbles(data))
    s = e4m3_decode(sf)
    shp = vals.shape
    return (vals.reshape(*shp[:-1], shp[-1] // 16, 16) * s[..., None]).reshape(shp).astype(f32)


def dequant_grouped_q(q_pack: np.ndarray, q_sf: np.ndarray, g: int):
    """(base, residue) float32 [B, Hkv, G, D] from the grouped-Q quantiser's outputs."""
    b, h, p, dh = q_pack.shape
    d = dh * 2
    vals = e2m1_decode(unpack_nibbles(q_pack))                        # [B,H,P,D]
    sf = np.asarray(q_sf, np.uint8).reshape(b * h, 128 * (d // 16))
    rows = np.arange(p)[:, None]
    lin = sf[:, sf_offset(rows, np.arange(d // 16)[None, :], d)].reshape(b, h, p, d // 16)
    deq = (vals.reshape(b, h, p, d // 16, 16) * e4m3_decode(lin)[..., None]).reshape(b, h, p, d)
    return deq[:, :, :g].astype(f32), deq[:, :, p // 2:p // 2 + g].astype(f32)


def _gather_tokens(cache: np.ndarray, block_table: np.ndarray, length: int, page: int):
    """cache [pages, H, page, D] -> [H, length, D] for one sequence."""
    n_pages = (length + page - 1) // page
    x = cache[block_table[:n_pages]]                                   # [n, H, page, D]
    x = np.transpose(x, (1, 0, 2, 3)).reshape(cache.shape[1], n_pages * page, cache.shape[3])
    return x[:, :length]


def resattn_decode_reference(q: np.ndarray, kv: dict, sm_scale: float, *, q_residue: bool = True,
                             p_e4m3: bool = False, v_e4m3: bool = False, rcp=None,
                             return_partials_for_splits: int = 0, tile: int = 256):
    """q float32 [B, Hq, D] (bf16-exact) -> bf16-rounded float32 [B, Hq, D].

    ``q_residue=False`` drops the residue rows (plain NVFP4 Q).  With
    ``return_partials_for_splits = S`` the function also returns the per-split (o, l, m) partials
    of the reference's strided split-KV schedule (sequence tiles of ``tile`` tokens dealt round
    robin to S splits, kernel_paged_decode.py:872-873) for testing the merge."""
    q = np.asarray(q, dtype=f32)
    b, hq, d = q.shape
    hkv = kv["k_data"].shape[1]
    g = hq // hkv
    page = kv["k_data"].shape[2]
    q_pack, q_sf = nvfp4_quant_grouped_q(q.reshape(b, hkv, g, d), rcp)
    qb, qr = dequant_grouped_q(q_pack, q_sf, g)
    kd = dequant_paged(kv["k_data"], kv["k_sf"])
    vd = dequant_paged(kv["v_data"], kv["v_sf"])
    if v_e4m3:
        vd = e4m3_encode(np.abs(vd))[1] * np.sign(vd)
    a = float(sm_scale) * float(kv["k_global_scale"])
    out = np.zeros((b, hq, d), dtype=np.float64)
    partials = []
    for i in range(b):
        length = int(kv["seq_lens"][i])
        if length == 0:
            continue
        kt = _gather_tokens(kd, kv["block_tables"][i], length, page).astype(np.float64)
        vt = _gather_tokens(vd, kv["block_tables"][i], length, page).astype(np.float64)
        s = np.einsum("hgd,htd->hgt", qb[i].astype(np.float64), kt)
        if q_residue:
            s = s + np.einsum("hgd,htd->hgt", qr[i].astype(np.float64), kt)
        s = s * a
        m = s.max(axis=-1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(axis=-1, keepdims=True)
        pq = e4m3_encode(p.astype(f32))[1].astype(np.float64) if p_e4m3 else p
        o = np.einsum("hgt,htd->hgd", pq, vt)
        out[i] = (o / l * float(kv["v_global_scale"])).reshape(hq, d)
        if return_partials_for_splits:
            sp = return_partials_for_splits
            tiles = (length + tile - 1) // tile
            for j in range(sp):
                idx = np.concatenate([np.arange(t * tile, min((t + 1) * tile, length))
                                      for t in range(j, tiles, sp)] or [np.zeros(0, np.int64)]).astype(np.int64)
                if idx.size == 0:
                    partials.append((i, j, None))
                    continue
                sj = s[:, :, idx]
                mj = sj.max(axis=-1, keepdims=True)
                pj = np.exp(sj - mj)
                partials.append((i, j, (np.einsum("hgt,htd->hgd", pj, vt[:, idx]).reshape(hq, d),
                                        pj.sum(axis=-1).reshape(hq), mj.reshape(hq))))
    res = bf16_round(out.astype(f32))
    return (res, partials) if return_partials_for_splits else res


def merge_splits(o_parts: np.ndarray, l_parts: np.ndarray, m_parts: np.ndarray, scale_o: float = 1.0):
    """Log-sum-exp merge of split-KV partials (natural-log domain):
    o = sum_i e^(m_i-m) o_i / sum_i e^(m_i-m) l_i * scale_o  (kernel_paged_decode.py:2822-2834).
    o_parts [S, ..., D]; l_parts, m_parts [S, ...]; empty splits carry l = 0, m = -inf."""
    m = np.max(m_parts, axis=0)
    with np.errstate(invalid="ignore"):
        w = np.where(np.isfinite(m_parts), np.exp(m_parts - m), 0.0)
    o = (w[..., None] * o_parts).sum(axis=0)
    l = (w * l_parts).sum(axis=0)
    return o / l[..., None] * scale_o


def quantize_attention_output_nvfp4(out: np.ndarray, global_scale, rcp=None):
    """Packed NVFP4 form of an attention output ``out`` [B, Hq, D] (float32): codes uint8 [B, Hq*D/2] and the
    128x4-swizzled E4M3 block-scale buffer over rows = sequences, hidden = Hq*D.

    Arithmetic of quantize_nvfp4_block16 / output_scale_offset (csrc/resattn/output.py:10-34): per 16
    consecutive values of the flattened hidden axis, scale = e4m3(amax * g * (1/6)) evaluated left to right
    in float32, multiplier = g * rcp(scale) (0 for an all-zero block), codes = e2m1(value * multiplier)."""
    from .fp4_codec import ExactRcp, e2m1_encode, e4m3_encode, pack_nibbles, swizzle_scales
    rcp = rcp or ExactRcp()
    b = out.shape[0]
    hidden = int(np.prod(out.shape[1:]))
    g = f32(global_scale)
    v = np.ascontiguousarray(out, dtype=f32).reshape(b, hidden // 16, 16)
    amax = np.abs(v).max(-1).astype(f32)
    sfv = ((amax * g).astype(f32) * f32(1.0 / 6.0)).astype(f32)
    sf_byte, sf_val = e4m3_encode(sfv)
    safe = np.where(sf_val != 0, sf_val, f32(1.0)).astype(f32)
    mult = np.where(sf_val != 0, (g * rcp(safe)).astype(f32), f32(0.0)).astype(f32)
    codes = e2m1_encode((v * mult[..., None]).astype(f32)).reshape(b, hidden)
    return pack_nibbles(codes), swizzle_scales(sf_byte.reshape(b, hidden // 16))
