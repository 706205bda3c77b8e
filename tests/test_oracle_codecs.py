"""Known-answer and property tests of the oracle's codecs and layouts (CPU)."""
import numpy as np
import pytest

import oracle as O


def test_e2m1_grid_and_ties():
    v = np.array([0, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.1, 7, 1e9, -0.1, -0.3, -6.5], np.float32)
    want = [0, 0, 0.5, 1, 1, 2, 2, 4, 4, 6, 6, 6, -0.0, -0.5, -6]
    got = O.e2m1_decode(O.e2m1_encode(v))
    assert np.array_equal(got, np.array(want, np.float32))
    assert O.e2m1_encode(np.array([-0.1], np.float32))[0] == 8          # sign kept on a zero result
    codes = np.arange(16, dtype=np.uint8)
    assert np.array_equal(O.e2m1_encode(O.e2m1_decode(codes)) & 7, codes & 7)


def test_nibble_packing_low_first():
    c = np.array([[1, 2, 3, 4]], np.uint8)
    p = O.pack_nibbles(c)
    assert p.tolist() == [[0x21, 0x43]]
    assert np.array_equal(O.unpack_nibbles(p), c)


def test_e4m3_roundtrip_and_saturation():
    allb = np.arange(0, 127, dtype=np.uint8)
    vals = O.e4m3_decode(allb)
    b, v = O.e4m3_encode(vals)
    assert np.array_equal(b, allb) and np.array_equal(v, vals)
    b, v = O.e4m3_encode(np.array([448, 460, 1e6, 2 ** -10, 2 ** -10 * 1.01, 0.0], np.float32))
    assert v.tolist() == [448, 448, 448, 0.0, 2 ** -9, 0.0]
    ml = pytest.importorskip("ml_dtypes")
    x = np.abs(np.random.default_rng(0).standard_normal(50000).astype(np.float32)) * 30
    assert np.array_equal(O.e4m3_encode(x)[0], np.minimum(x, 448).astype(ml.float8_e4m3fn).view(np.uint8))


def test_e8m0_ceil():
    v = np.array([0, 1, 1.0001, 0.5, 0.75, 6, 3e38], np.float32)
    assert O.e8m0_ceil_encode(v).tolist() == [0, 127, 128, 126, 127, 130, 254]
    assert O.e8m0_decode(np.array([127, 130], np.uint8)).tolist() == [1.0, 8.0]


def test_swizzle_layout_formula_and_roundtrip():
    lin = np.random.default_rng(0).integers(0, 255, (200, 24), dtype=np.uint8)
    sw = O.swizzle_scales(lin)
    assert sw.size == 2 * 6 * 512
    # byte offset formula of the 128x4 layout
    m, g = 130, 9
    off = (m // 128) * (6 * 512) + (g // 4) * 512 + (m % 32) * 16 + ((m % 128) // 32) * 4 + g % 4
    assert sw[off] == lin[m, g]
    assert np.array_equal(O.unswizzle_scales(sw, 200, 24), lin)


def test_bf16_helpers():
    x = np.array([1.0, 1.00390625, 1.0 + 2 ** -9, 3.14159], np.float32)
    r = O.bf16_round(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == 1.0      # 2^-8 and 2^-9 steps round to 1.0 (tie to even)
    assert np.array_equal(O.from_bf16_bits(O.to_bf16_bits(r)), r)
    assert O.bf16_round(np.array([1.0 + 2 ** -8], np.float32))[0] == 1.0       # tie to even


@pytest.mark.parametrize("layout", range(5))
def test_mext_layout_row_maps(layout):
    m, k = 11, 64
    x = O.make_activation(m, k, seed=3)
    codes, sf, written = O.nvfp4_quant_mext(x, np.float32(100.0), layout)
    q = O.nvfp4_mext_blocks(np.vstack([x, np.zeros((5 if layout in (2, 4) else 0, k), np.float32)]), np.float32(100.0))
    i = 9
    if layout == 3:
        assert codes.shape == (m, k)
        assert np.array_equal(codes[i, :k // 2], O.pack_nibbles(q["base_codes"])[i])
        assert np.array_equal(codes[i, k // 2:], O.pack_nibbles(q["res_codes"])[i])
    else:
        base = {0: i, 1: 2 * i, 2: 16 + 1, 4: 16 + 1}[layout]
        res = {0: i + m, 1: 2 * i + 1, 2: 16 + 9, 4: 16 + 9}[layout]
        assert np.array_equal(codes[base], O.pack_nibbles(q["base_codes"])[i])
        assert np.array_equal(codes[res], O.pack_nibbles(q["res_codes"])[i])
    assert written.any() and sf.size == written.size


def test_residue_reduces_error():
    """deq(q(x)) + deq(q(r)) is closer to x than deq(q(x)) alone (the point of MEXT)."""
    x = O.make_activation(8, 256, seed=1)
    gi = np.float32(6 * 448) / np.abs(x).max()
    q = O.nvfp4_mext_blocks(x, gi)
    base = O.nvfp4_dequant(O.pack_nibbles(q["base_codes"]), q["base_sf"], 1 / gi)
    res = O.nvfp4_dequant(O.pack_nibbles(q["res_codes"]), q["res_sf"], 1 / gi)
    e0 = np.linalg.norm(x - base)
    e1 = np.linalg.norm(x - base - res)
    assert e1 < 0.35 * e0


def test_kext_residue_order_and_scale_groups():
    m, k, per8 = 2, 256, 2
    x = O.make_activation(m, k, seed=5)
    mask = O.make_kext_mask(k, per8)
    sel = O.mask_to_indices(mask)
    assert sel.size == k // 4 and np.all(np.diff(sel) > 0)
    assert all(bin(b).count("1") == per8 for b in mask)
    codes, sf, written = O.nvfp4_quant_kext(x, np.float32(50.0), mask, per8)
    assert codes.shape == (m, (k + sel.size) // 2)
    # rows up to 128 have defined (zero) scales
    assert written.sum() == 128 * (k + sel.size) // 16
    lin = O.unswizzle_scales(sf, 128, (k + sel.size) // 16)
    assert not lin[m:].any()


def test_mxfp4_blocks_power_of_two_scale():
    x = O.make_activation(4, 128, seed=2)
    codes, e, deq = O.mxfp4_blocks(x.reshape(4, 4, 32))
    amax = np.abs(x.reshape(4, 4, 32)).max(-1)
    scale = O.e8m0_decode(e)
    assert np.all(scale * 6 >= amax * (1 - 1e-6)) and np.all(scale * 3 < amax * (1 + 1e-6) + 1e-30)
    assert np.abs(deq - x.reshape(4, 4, 32)).max() <= scale.max() * 1.0


def test_config0_mext_linear_on_cpu():
    """The reference's CPU-runnable configuration (x [16, 5120], reduced N for speed): the folded contraction equals the two-term sum and
    tracks the torch-eager reference path."""
    import torch
    m, k, n = 16, 5120, 512
    x, w = O.make_activation(m, k, seed=0), O.make_weight(n, k, seed=1)
    gx = np.float32(np.abs(x).max() / (6 * 448))
    gw = np.float32(np.abs(w).max() / (6 * 448))
    codes, sf, _ = O.nvfp4_quant_mext(x, np.float32(1) / gx, O.LAYOUT_ROW_PAIR)
    a = O.dequant_operand(codes, sf, "nvfp4")
    wc, wsf = O.nvfp4_quant_plain(w, np.float32(1) / gw)
    wd = O.dequant_operand(wc, wsf, "nvfp4")
    alpha = float(gx) * float(gw)
    y_fold = O.fp4_linear_reference(a[0::2] + a[1::2], wd, alpha, round_bf16=False)
    y_two = O.fp4_linear_reference(a[0::2], wd, alpha, False) + O.fp4_linear_reference(a[1::2], wd, alpha, False)
    assert np.allclose(y_fold, y_two, rtol=1e-5, atol=1e-6)
    y_eager = O.eager_residue_linear(torch.from_numpy(x), torch.from_numpy(w), out_dtype=torch.float32).numpy()
    y_exact = x.astype(np.float64) @ w.astype(np.float64).T
    rel = lambda a_, b_: np.linalg.norm(a_ - b_) / np.linalg.norm(b_)
    assert rel(y_fold, y_eager) < 0.02           # same recipe up to reciprocal / rounding details
    assert rel(y_fold, y_exact) < 0.15           # W4A4 quantisation error level


def test_resattn_oracle_partials_merge():
    kv = O.make_paged_kv([300, 40], 2, 128, 16, seed=1)
    q = O.bf16_round(np.random.default_rng(0).standard_normal((2, 16, 128)).astype(np.float32))
    ref, parts = O.resattn_decode_reference(q, kv, 128 ** -0.5, return_partials_for_splits=3, tile=64)
    for b in range(2):
        o = np.zeros((3, 16, 128)); l = np.zeros((3, 16)); mm = np.full((3, 16), -np.inf)
        for (bi, j, p) in parts:
            if bi == b and p is not None:
                o[j], l[j], mm[j] = p
        merged = O.merge_splits(o, l, mm, kv["v_global_scale"])
        assert np.allclose(O.bf16_round(merged.astype(np.float32)), ref[b], rtol=2e-2, atol=1e-3)
    # the residue improves on plain NVFP4 Q
    exact_q = O.resattn_decode_reference(q, kv, 128 ** -0.5)
    no_res = O.resattn_decode_reference(q, kv, 128 ** -0.5, q_residue=False)
    assert np.abs(no_res - exact_q).max() > 0
