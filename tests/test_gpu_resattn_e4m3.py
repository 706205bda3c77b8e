"""ResAttn decode with V and P in E4M3 (``ops.resattn_pv_format("e4m3")``), the number format of the reference's own
kernel (csrc/resattn/kernel_paged_decode.py:1958-1963, csrc/resattn/qmul4.py:45).

The oracle's E4M3 mode rounds the dequantised V and the probabilities exactly where the reference does.  The kernel
rounds V identically (code x block scale is exact in FP16, then round-to-nearest-even, saturating); its probabilities
are taken against a running maximum instead of the final one, so they round differently and the comparison is a
tolerance: the kernel must sit about as close to the E4M3-mode oracle as that oracle sits to exact attention (within
1.25 x), and no further from exact attention than 1.5 x that distance.  Caches are FP8-range (global scale amax / 448), where the
E4M3 expansion of V cannot saturate."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _run(dev, kv, q_np, sm, splits, fmt):
    from resinfer_b200 import ops
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)      # noqa: E731
    b, hq, d = q_np.shape
    out = torch.zeros(b, hq, d, dtype=torch.float32, device=dev)
    with ops.resattn_pv_format(fmt):
        ops.resattn_decode(t(q_np).to(torch.bfloat16), t(kv["k_data"]), t(kv["k_sf"]), t(kv["v_data"]), t(kv["v_sf"]),
                           t(np.maximum(kv["block_tables"], 0)), t(kv["seq_lens"]), sm * kv["k_global_scale"],
                           kv["v_global_scale"], out, splits=splits)
    torch.cuda.synchronize()
    ops.check_status(dev)
    return out.cpu().numpy()


@pytest.mark.parametrize("d,page,lens,hkv,g,splits", [
    (128, 16, [3000, 1200, 257], 2, 8, 2), (128, 128, [500, 129, 4000], 1, 8, 3), (256, 16, [300, 64, 2500], 2, 8, 1),
    (256, 128, [1000, 2049], 1, 6, 4), (128, 16, [1, 16, 17, 0], 2, 4, 2)])
def test_e4m3_format_matches_the_reference_rounding(cuda_device, device_rcp, d, page, lens, hkv, g, splits):
    kv = O.make_paged_kv(lens, hkv, d, page, seed=d + page, scale_range=448.0)
    q_np = O.bf16_round(np.random.default_rng(6).standard_normal((len(lens), hkv * g, d)).astype(np.float32))
    sm = d ** -0.5
    rcp = O.RecordingRcp(device_rcp)
    exact = O.resattn_decode_reference(q_np, kv, sm, rcp=rcp)
    e4m3 = O.resattn_decode_reference(q_np, kv, sm, rcp=rcp, p_e4m3=True, v_e4m3=True)
    got = _run(cuda_device, kv, q_np, sm, splits, "e4m3")
    fp16 = _run(cuda_device, kv, q_np, sm, splits, "fp16")
    assert np.isfinite(got).all()
    d_exact, d_ref, d_round = rel_fro(got, exact), rel_fro(got, e4m3), rel_fro(e4m3, exact)
    print(f"e4m3 kernel vs exact {d_exact:.3e}; vs E4M3-mode oracle {d_ref:.3e}; E4M3-mode oracle vs exact {d_round:.3e}; "
          f"fp16 kernel vs exact {rel_fro(fp16, exact):.3e}")
    assert d_ref < 1.25 * d_round + 3e-3
    assert d_exact < 1.5 * d_round + 3e-3
    assert d_exact > 2 * rel_fro(fp16, exact)                  # the format switch is really on
    for i, L in enumerate(lens):
        if L == 0:
            assert not got[i].any()


def test_e4m3_format_at_a_benchmark_shape(cuda_device):
    """64 query heads, 8 KV heads, batch 16 with ragged contexts up to 8192, pages of 128 tokens (the copy-engine path),
    6 splits: splits and block-table permutations change nothing but the summation order."""
    from resinfer_b200 import ops
    dev = cuda_device
    d, hq, hkv, page, b = 128, 64, 8, 128, 16
    g = torch.Generator(device=dev).manual_seed(1)
    lens = torch.randint(100, 8193, (b,), generator=g, device=dev, dtype=torch.int32)
    pages_per = (lens + page - 1) // page
    total = int(pages_per.sum())
    perm = torch.randperm(total + 7, generator=g, device=dev)[:total].to(torch.int32)
    bt = torch.zeros(b, int(pages_per.max()), dtype=torch.int32, device=dev)
    off = 0
    for i in range(b):
        n = int(pages_per[i])
        bt[i, :n] = perm[off:off + n]
        off += n
    pool = total + 7
    kd = torch.randint(0, 256, (pool, hkv, page, d // 2), generator=g, device=dev, dtype=torch.uint8)
    # V codes without sign bits: sums of same-sign terms, so rounding errors average instead of being divided by a
    # small difference of large sums
    vd = torch.randint(0, 256, (pool, hkv, page, d // 2), generator=g, device=dev, dtype=torch.uint8) & 0x77
    ks = torch.randint(0x28, 0x40, (pool, hkv, page, d // 16), generator=g, device=dev, dtype=torch.uint8)
    vs = torch.randint(0x28, 0x40, (pool, hkv, page, d // 16), generator=g, device=dev, dtype=torch.uint8)
    q = torch.randn(b, hq, d, generator=g, device=dev).to(torch.bfloat16)
    outs = {}
    for fmt, splits in (("fp16", 1), ("e4m3", 1), ("e4m3", 6)):
        o = torch.zeros(b, hq, d, dtype=torch.float32, device=dev)
        with ops.resattn_pv_format(fmt):
            ops.resattn_decode(q, kd, ks, vd, vs, bt, lens, 0.01, 1.0, o, splits=splits)
        torch.cuda.synchronize()
        ops.check_status(dev)
        outs[(fmt, splits)] = o
    ref = outs[("fp16", 1)]
    err = lambda a: float((a - ref).norm() / ref.norm())         # noqa: E731
    assert torch.isfinite(outs[("e4m3", 1)]).all()
    assert 1e-3 < err(outs[("e4m3", 1)]) < 8e-2
    assert float((outs[("e4m3", 6)] - outs[("e4m3", 1)]).norm() / ref.norm()) < 2e-2
