"""GPU parity of ResAttn decode against the CPU oracle (exact attention over the dequantised NVFP4 KV
cache with the NVFP4 + residue query).  The reference kernel itself cannot be built on this toolchain,
so this parity is a tolerance, not a bit-exact pin: FP32 output within 1e-3 relative Frobenius error (P is
rounded to FP16 before the PV product), BF16 output within BF16 rounding."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_BF16 = 3e-3


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _run(dev, kv, q_np, sm, splits, out_dtype=torch.float32, q_residue=True, want_q=False):
    from resinfer_b200 import ops
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    b, hq, d = q_np.shape
    hkv = kv["k_data"].shape[1]
    out = torch.zeros(b, hq, d, dtype=out_dtype, device=dev)
    qp = qs = None
    if want_q:
        p = 8 if hq // hkv == 4 else 16
        qp = torch.zeros(b, hkv, p, d // 2, dtype=torch.uint8, device=dev)
        qs = torch.zeros(b * hkv * 128 * d // 16, dtype=torch.uint8, device=dev)
    ops.resattn_decode(t(q_np).to(torch.bfloat16), t(kv["k_data"]), t(kv["k_sf"]), t(kv["v_data"]), t(kv["v_sf"]),
                       t(np.maximum(kv["block_tables"], 0)), t(kv["seq_lens"]), sm * kv["k_global_scale"],
                       kv["v_global_scale"], out, splits=splits, q_residue=q_residue, q_pack=qp, q_sf=qs)
    torch.cuda.synchronize()
    ops.check_status(dev)
    return out, qp, qs


@pytest.mark.parametrize("d,page,lens,hkv,g,splits", [
    (128, 16, [100, 777], 2, 8, 1), (128, 16, [1, 16, 17, 3000], 2, 8, 4), (128, 128, [500, 129], 1, 8, 2),
    (256, 16, [300, 64], 2, 8, 1), (128, 16, [333], 2, 4, 3), (256, 32, [1000], 1, 6, 5),
    (128, 64, [2049, 5], 8, 8, 8), (128, 16, [0, 50], 1, 8, 2)])
def test_decode_matches_oracle(cuda_device, device_rcp, d, page, lens, hkv, g, splits):
    kv = O.make_paged_kv(lens, hkv, d, page, seed=d + page)
    b, hq = len(lens), hkv * g
    q_np = O.bf16_round(np.random.default_rng(9).standard_normal((b, hq, d)).astype(np.float32))
    sm = d ** -0.5
    ref = O.resattn_decode_reference(q_np, kv, sm, rcp=O.RecordingRcp(device_rcp))
    ref32 = ref                                              # oracle output is BF16-rounded
    out32, qp, qs = _run(cuda_device, kv, q_np, sm, splits, want_q=True)
    got = out32.cpu().numpy()
    assert not np.isnan(got).any()
    assert rel_fro(got, ref32) < TOL_BF16                     # vs the BF16-rounded oracle
    out16, _, _ = _run(cuda_device, kv, q_np, sm, splits, out_dtype=torch.bfloat16)
    assert torch.equal(out16, out32.to(torch.bfloat16))
    # the fused query quantiser is bit-identical to the grouped-Q quantiser
    op, osf = O.nvfp4_quant_grouped_q(q_np.reshape(b, hkv, g, d), rcp=O.RecordingRcp(device_rcp))
    assert np.array_equal(qp.cpu().numpy(), op) and np.array_equal(qs.cpu().numpy(), osf)
    for i, L in enumerate(lens):
        if L == 0:
            assert not got[i].any()                           # empty sequence -> zeros


def test_decode_unrounded_accuracy_and_residue_effect(cuda_device, device_rcp):
    """FP32 output against a float64 oracle without output rounding; dropping the query residue moves
    the result measurably away (the compensation is real), and split counts agree with each other."""
    d, page, hkv, g = 128, 16, 2, 8
    lens = [4097, 900]
    kv = O.make_paged_kv(lens, hkv, d, page, seed=5)
    q_np = O.bf16_round(np.random.default_rng(2).standard_normal((2, hkv * g, d)).astype(np.float32))
    sm = d ** -0.5
    # unrounded oracle: recompute in float64 from the oracle's pieces
    qpk, qsf = O.nvfp4_quant_grouped_q(q_np.reshape(2, hkv, g, d), rcp=O.RecordingRcp(device_rcp))
    qb, qr = O.dequant_grouped_q(qpk, qsf, g)
    kd, vd = O.dequant_paged(kv["k_data"], kv["k_sf"]), O.dequant_paged(kv["v_data"], kv["v_sf"])
    exact = np.zeros((2, hkv * g, d))
    plain = np.zeros_like(exact)
    for i, L in enumerate(lens):
        n = (L + page - 1) // page
        pages = kv["block_tables"][i, :n]
        k = kd[pages].transpose(1, 0, 2, 3).reshape(hkv, n * page, d)[:, :L].astype(np.float64)
        v = vd[pages].transpose(1, 0, 2, 3).reshape(hkv, n * page, d)[:, :L].astype(np.float64)
        for qq, dst in (((qb[i] + qr[i]).astype(np.float64), exact), (qb[i].astype(np.float64), plain)):
            s = np.einsum("hgd,htd->hgt", qq, k) * sm * kv["k_global_scale"]
            p = np.exp(s - s.max(-1, keepdims=True))
            dst[i] = (np.einsum("hgt,htd->hgd", p, v) / p.sum(-1, keepdims=True) * kv["v_global_scale"]).reshape(-1, d)
    o1, _, _ = _run(cuda_device, kv, q_np, sm, 1)
    o8, _, _ = _run(cuda_device, kv, q_np, sm, 8)
    assert rel_fro(o1.cpu().numpy(), exact) < TOL_F32
    assert rel_fro(o8.cpu().numpy(), exact) < TOL_F32
    assert rel_fro(o8.cpu().numpy(), o1.cpu().numpy()) < TOL_F32
    nores, _, _ = _run(cuda_device, kv, q_np, sm, 1, q_residue=False)
    assert rel_fro(nores.cpu().numpy(), plain) < TOL_F32
    assert rel_fro(nores.cpu().numpy(), exact) > 5 * rel_fro(o1.cpu().numpy(), exact)


def test_reference_named_host_entry(cuda_device):
    from resinfer_b200.nvfp4.cute_attn.host import (allocate_qmul4_reduction_workspace, plan_qmul4_decode,
                                                     run_paged_fp4_decode_qmul4_tmem)
    from resinfer_b200.nvfp4.cute_attn.kv_layout import NvFp4PagedKVPool
    d, page, hkv, g = 128, 128, 2, 8
    lens = [700, 1300, 128]
    kv = O.make_paged_kv(lens, hkv, d, page, seed=11)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    q_np = O.bf16_round(np.random.default_rng(3).standard_normal((3, hkv * g, d)).astype(np.float32))
    pool = NvFp4PagedKVPool(hkv, d, t(kv["k_data"]), t(kv["v_data"]), t(kv["k_sf"]), t(kv["v_sf"]), page_size=page,
                            k_global_scale=kv["k_global_scale"], v_global_scale=kv["v_global_scale"])
    q = t(q_np).to(torch.bfloat16)
    out = torch.empty(3, hkv * g, d, dtype=torch.bfloat16, device=cuda_device)
    bt, sl = t(np.maximum(kv["block_tables"], 0)), t(kv["seq_lens"])
    plan = plan_qmul4_decode(3, hkv, 1300, cuda_device, head_dim=d)
    ws = allocate_qmul4_reduction_workspace(4, 3, hkv * g, d, cuda_device)
    for pl, w in ((None, None), (plan, None), ((4, "kernel"), ws), ((1, "none"), None)):
        out.zero_()
        run_paged_fp4_decode_qmul4_tmem(q, pool, pool.v_data, pool.v_sf, bt, sl, d ** -0.5 * pool.k_global_scale, out,
                                        value_scale=pool.v_global_scale, plan=pl, reduction_workspace=w)
        ref = O.resattn_decode_reference(q_np, kv, d ** -0.5)
        assert rel_fro(out.float().cpu().numpy(), ref) < TOL_BF16
    with pytest.raises(ValueError, match="seq_lens"):
        run_paged_fp4_decode_qmul4_tmem(q, pool, pool.v_data, pool.v_sf, bt, sl.long(), 0.1, out)
    with pytest.raises(ValueError, match="v_data_hnd"):
        run_paged_fp4_decode_qmul4_tmem(q, pool, pool.v_data[:, :1], pool.v_sf, bt, sl, 0.1, out)
    with pytest.raises(NotImplementedError):
        run_paged_fp4_decode_qmul4_tmem(q, pool, pool.v_data, pool.v_sf, bt, sl, 0.1, out, residue_fold=False)
    with pytest.raises(ValueError, match="BF16"):
        run_paged_fp4_decode_qmul4_tmem(q, pool, pool.v_data, pool.v_sf, bt, sl, 0.1, out.float())


def test_decode_at_baseline_shape(cuda_device):
    """The benchmarked shape (64 query heads, 8 KV heads, page 16, contexts up to 32768) with random KV bytes:
    properties only -- finite output, split invariance, and permuting the page pool together with the
    block table leaves the result unchanged."""
    from resinfer_b200 import ops
    b, hq, hkv, d, page = 4, 64, 8, 128, 16
    g = torch.Generator(device=cuda_device).manual_seed(0)
    lens = torch.tensor([32768, 1024, 20000, 9999], dtype=torch.int32, device=cuda_device)
    per = (lens + page - 1) // page
    pool = int(per.sum()) + 7
    perm = torch.randperm(pool, generator=g, device=cuda_device).to(torch.int32)
    bt = torch.zeros(b, int(per.max()), dtype=torch.int32, device=cuda_device)
    off = 0
    for i in range(b):
        bt[i, :int(per[i])] = perm[off:off + int(per[i])]
        off += int(per[i])
    rnd = lambda *s, lo=0, hi=256: torch.randint(lo, hi, s, generator=g, device=cuda_device, dtype=torch.uint8)
    kd, vd = rnd(pool, hkv, page, d // 2), rnd(pool, hkv, page, d // 2)
    ks, vs = rnd(pool, hkv, page, d // 16, lo=0x30, hi=0x40), rnd(pool, hkv, page, d // 16, lo=0x30, hi=0x40)
    q = torch.randn(b, hq, d, generator=g, device=cuda_device).to(torch.bfloat16)
    run = lambda kd_, ks_, vd_, vs_, bt_, s: ops.resattn_decode(
        q, kd_, ks_, vd_, vs_, bt_, lens, d ** -0.5, 1.0, torch.empty(b, hq, d, dtype=torch.float32, device=cuda_device),
        splits=s)
    o1, o16 = run(kd, ks, vd, vs, bt, 1), run(kd, ks, vd, vs, bt, 16)
    assert torch.isfinite(o1).all()
    assert rel_fro(o16.cpu().numpy(), o1.cpu().numpy()) < TOL_F32
    shuffle = torch.randperm(pool, generator=g, device=cuda_device)
    inv = torch.empty_like(shuffle)
    inv[shuffle] = torch.arange(pool, device=cuda_device)
    o_perm = run(kd[shuffle], ks[shuffle], vd[shuffle], vs[shuffle], inv[bt.long()].to(torch.int32), 16)
    assert torch.equal(o_perm, o16)
    torch.cuda.synchronize()
    ops.check_status(cuda_device)


@pytest.mark.parametrize("lens,splits", [([100, 777, 16], 1), ([3000, 5, 700], 4)])
def test_decode_nvfp4_output(cuda_device, device_rcp, lens, splits):
    """Packed NVFP4 output: the codes and block scales equal the oracle's quantisation of the kernel's own
    unrounded output bit for bit, through the reference-named host entry as well."""
    from resinfer_b200 import ops
    from resinfer_b200.nvfp4.cute_attn.host import (allocate_nvfp4_attention_output,
                                                     run_paged_fp4_decode_qmul4_tmem_nvfp4)
    from resinfer_b200.nvfp4.cute_attn.kv_layout import NvFp4PagedKVPool
    d, page, hkv, g = 128, 16, 2, 8
    kv = O.make_paged_kv(lens, hkv, d, page, seed=21)
    b, hq = len(lens), hkv * g
    q_np = O.bf16_round(np.random.default_rng(4).standard_normal((b, hq, d)).astype(np.float32))
    sm = d ** -0.5
    out32, _, _ = _run(cuda_device, kv, q_np, sm, splits)
    gs = 6.0 * 448.0 / float(out32.abs().max())
    want_codes, want_sf = O.quantize_attention_output_nvfp4(out32.cpu().numpy(), gs, rcp=O.RecordingRcp(device_rcp))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    gsi = torch.tensor([gs], dtype=torch.float32, device=cuda_device)
    pool = NvFp4PagedKVPool(hkv, d, t(kv["k_data"]), t(kv["v_data"]), t(kv["k_sf"]), t(kv["v_sf"]), page_size=page,
                            k_global_scale=kv["k_global_scale"], v_global_scale=kv["v_global_scale"])
    codes, sf = run_paged_fp4_decode_qmul4_tmem_nvfp4(
        t(q_np).to(torch.bfloat16), pool, pool.v_data, pool.v_sf, t(np.maximum(kv["block_tables"], 0)),
        t(kv["seq_lens"]), sm * pool.k_global_scale, gsi, value_scale=pool.v_global_scale, plan=(splits, "kernel" if splits > 1 else "none"))
    torch.cuda.synchronize()
    ops.check_status(cuda_device)
    assert codes.shape == (b, hq * d // 2) and sf.dtype == torch.float8_e4m3fn
    assert np.array_equal(codes.cpu().numpy(), want_codes)
    got_sf = sf.view(torch.uint8).reshape(-1).cpu().numpy()
    # rows beyond the batch are never written (the buffer starts zeroed): compare the rows that exist
    hidden = hq * d
    for row in range(b):
        for blk in range(0, hidden // 16, 37):
            off = O.sf_offset(row, blk, hidden)
            assert got_sf[off] == want_sf[off]
    # dequantised output stays within FP4 error of the unrounded one
    deq = O.nvfp4_dequant(codes.cpu().numpy(), O.unswizzle_scales(got_sf, b, hidden // 16), 1.0 / gs)
    assert rel_fro(deq, out32.cpu().numpy().reshape(b, -1)) < 0.12
    out_b, sf_b = allocate_nvfp4_attention_output(b, hq, d, cuda_device)
    with pytest.raises(ValueError, match="supplied together"):
        run_paged_fp4_decode_qmul4_tmem_nvfp4(t(q_np).to(torch.bfloat16), pool, pool.v_data, pool.v_sf,
                                              t(np.maximum(kv["block_tables"], 0)), t(kv["seq_lens"]), 0.1, gsi, out=out_b)
    with pytest.raises(ValueError, match="one-element"):
        run_paged_fp4_decode_qmul4_tmem_nvfp4(t(q_np).to(torch.bfloat16), pool, pool.v_data, pool.v_sf,
                                              t(np.maximum(kv["block_tables"], 0)), t(kv["seq_lens"]), 0.1,
                                              torch.ones(2, device=cuda_device), out=out_b, output_block_scale=sf_b)


@pytest.mark.parametrize("d,splits", [(128, 1), (128, 2), (256, 1), (256, 3)])
def test_decode_late_maxima_rescale_accumulators(cuda_device, device_rcp, d, splits):
    """Scores that grow along the sequence: the K block scales of later 128-token tiles are raised by a
    few E4M3 exponent steps, so the running maximum of every head moves by far more than the lazy
    threshold (2^8) on several tiles after the first one and the accumulated P.V has to be rescaled in
    place each time.  Checked against the oracle like every other case."""
    page, hkv, g = 16, 2, 8
    lens = [1500, 700]
    kv = O.make_paged_kv(lens, hkv, d, page, seed=11)
    ks = kv["k_sf"].copy()
    for b, L in enumerate(lens):
        for t in range(L):
            bump = (t // 128) // 2                           # 0, 0, 1, 1, 2, 2, ... exponent steps of 2 each
            if bump:
                pg = kv["block_tables"][b, t // page]
                row = ks[pg, :, t % page, :].astype(np.int32)
                ks[pg, :, t % page, :] = np.minimum(row + 16 * bump, 0x7E).astype(np.uint8)   # E4M3: +16 = x4
    kv["k_sf"] = ks
    b, hq = len(lens), hkv * g
    q_np = O.bf16_round((4.0 * np.random.default_rng(5).standard_normal((b, hq, d))).astype(np.float32))
    sm = d ** -0.5
    ref = O.resattn_decode_reference(q_np, kv, sm, rcp=O.RecordingRcp(device_rcp))
    out32, _, _ = _run(cuda_device, kv, q_np, sm, splits)
    got = out32.cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_fro(got, ref) < TOL_BF16


@pytest.mark.parametrize("d,page", [(128, 16), (256, 16), (128, 128)])
def test_decode_batch32_matches_oracle(cuda_device, device_rcp, d, page):
    """Batch 32 with short, ragged contexts (including an empty sequence and exact tile / page multiples):
    batch indexing, block-table row strides and per-sequence lengths beyond a handful of sequences."""
    hkv, g = 2, 8
    rng = np.random.default_rng(32)
    lens = [int(v) for v in rng.integers(1, 700, size=32)]
    lens[3], lens[7], lens[11], lens[30] = 0, 128, 256, 129
    kv = O.make_paged_kv(lens, hkv, d, page, seed=77)
    b, hq = len(lens), hkv * g
    q_np = O.bf16_round(rng.standard_normal((b, hq, d)).astype(np.float32))
    sm = d ** -0.5
    ref = O.resattn_decode_reference(q_np, kv, sm, rcp=O.RecordingRcp(device_rcp))
    for splits in (1, 3):
        out32, _, _ = _run(cuda_device, kv, q_np, sm, splits)
        got = out32.cpu().numpy()
        assert np.isfinite(got).all()
        assert rel_fro(got, ref) < TOL_BF16
        # per sequence as well: one wrong row of the block table must not hide among 31 right ones
        for i, L in enumerate(lens):
            if L == 0:
                assert not got[i].any()
            else:
                assert rel_fro(got[i], ref[i]) < 2 * TOL_BF16, (i, L)


def test_distance_from_exact_and_from_reference_rounding(cuda_device, device_rcp):
    """Where the kernel's numerics sit.  The reference kernel rounds P and the dequantised V to E4M3 before
    its FP8 P.V product (csrc/resattn/kernel_paged_decode.py:1958-1963, qmul4.py:45); this kernel keeps V
    exact (FP4 code x E4M3 scale fits FP16) and P in FP16.  Against the exact attention over the
    dequantised cache the kernel must therefore be much closer than the oracle run with the reference's
    E4M3 rounding is, and its distance from that E4M3-mode oracle must equal the rounding's own distance
    from exact (the kernel adds nothing measurable on top).  The three numbers are printed (-s)."""
    d, page, hkv, g = 128, 16, 2, 8
    lens = [3000, 1200, 257]
    # FP8-range cache (global scale amax/448): the E4M3 expansion of V then never saturates
    kv = O.make_paged_kv(lens, hkv, d, page, seed=9, scale_range=448.0)
    q_np = O.bf16_round(np.random.default_rng(6).standard_normal((len(lens), hkv * g, d)).astype(np.float32))
    sm = d ** -0.5
    rcp = O.RecordingRcp(device_rcp)
    exact = O.resattn_decode_reference(q_np, kv, sm, rcp=rcp)
    e4m3 = O.resattn_decode_reference(q_np, kv, sm, rcp=rcp, p_e4m3=True, v_e4m3=True)
    out32, _, _ = _run(cuda_device, kv, q_np, sm, 2)
    got = out32.cpu().numpy()
    d_exact, d_e4m3, d_round = rel_fro(got, exact), rel_fro(got, e4m3), rel_fro(e4m3, exact)
    print(f"kernel vs exact {d_exact:.3e}; kernel vs E4M3-mode oracle {d_e4m3:.3e}; E4M3-mode vs exact {d_round:.3e}")
    assert d_exact < TOL_BF16
    assert d_exact < 0.5 * d_round
    assert abs(d_e4m3 - d_round) < 0.25 * d_round + TOL_BF16
