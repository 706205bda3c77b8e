"""Speed of this library's quantisers beside the reference project's own sm_100 quantiser kernels on the same
GPU (``oracle/_ref/libnvfp4_ref.so``: the reference's .cu files compiled as they are; bit-identical outputs
are what ``tests/test_gpu_quant.py`` checks).  Microseconds per launch inside a CUDA graph of 20 back-to-back
launches, CUDA events around 5 replays after 3 warm-up replays.

Covers the NVFP4 MEXT quantiser (row_pair), the NVFP4 KEXT quantiser at residue ratios 0.125 / 0.25 / 0.5 and
the MXFP4 MEXT quantiser, at decode and prefill token counts for K = 5120, 8192, 25600.  The table is printed
(run with ``-s``) and, when the environment variable ``RESINFER_B200_REPORT_DIR`` names a directory, written there as
``quantisers_vs_reference.json``.  The assertion is deliberately loose (a launch must not take more than
1.6 x the reference kernel's time, plus 0.3 us): it guards against regressions, the numbers are the product.

One difference matters at decode sizes.  This library's quantisers wait for the kernel before them
(``griddepcontrol.wait``) because their input is usually that kernel's output, and let the kernel behind them
start early; the reference's MEXT quantiser never waits and only signals completion at its end.  In a chain of
identical launches with programmatic serialisation the reference kernel therefore skips the hand-over that a
dependent launch needs.  The MEXT rows are measured both ways: with programmatic launch (``ours_us`` /
``ref_us``) and with plain stream order (``*_plain_us``), where both kernels pay the same launch sequence.

    python -m pytest tests/test_gpu_quant_speed_vs_reference.py -s -q
"""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KS = (5120, 8192, 25600)
MS = (1, 16, 128, 1024, 8192)


def _time(fn, reps=20):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / 5 / reps


def test_quantisers_beside_the_reference_kernels(cuda_device, ref_ops):
    if ref_ops is None:
        pytest.skip("oracle/_ref/libnvfp4_ref.so is not built")
    from resinfer_b200.nvfp4.quant import indices_to_channel_masks
    from resinfer_b200.quant import weight_prep
    dev = cuda_device
    ours_ops = torch.ops.nvfp4
    rows = []
    for k in KS:
        for m in MS:
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            gi = torch.tensor([100.0], device=dev)
            # ---- NVFP4 MEXT, row_pair
            codes = torch.empty(2 * m * k // 2, dtype=torch.uint8, device=dev)
            sf = torch.zeros(((2 * m + 127) // 128) * ((k + 63) // 64) * 512, dtype=torch.uint8, device=dev)
            a = _time(lambda: ours_ops.scaled_fp4_quant_mext_r1(codes, x, sf, gi, 0, 1, True))
            b = _time(lambda: ref_ops.scaled_fp4_quant_mext_r1(codes, x, sf, gi, 0, 1, True))
            a0 = _time(lambda: ours_ops.scaled_fp4_quant_mext_r1(codes, x, sf, gi, 0, 1, False))
            b0 = _time(lambda: ref_ops.scaled_fp4_quant_mext_r1(codes, x, sf, gi, 0, 1, False))
            rows.append(dict(kernel="nvfp4_mext", k=k, m=m, ours_us=round(a, 2), ref_us=round(b, 2),
                             ours_plain_us=round(a0, 2), ref_plain_us=round(b0, 2),
                             ours_gbs=round((2 * m * k + 2 * m * k * 0.5625) / a / 1e3)))
            # ---- NVFP4 KEXT
            for per8, ratio in ((1, 0.125), (2, 0.25), (4, 0.5)):
                if m in (16, 1024):
                    continue                                   # keep the run short: decode, M = 128, long prefill
                idx = weight_prep.salient_indices_per8(k, per8, device=dev)
                mask = indices_to_channel_masks(idx, k)
                n_ext = k + idx.numel()
                kc = torch.empty(m * n_ext // 2, dtype=torch.uint8, device=dev)
                ks = torch.zeros(((m + 127) // 128) * ((n_ext + 63) // 64) * 512, dtype=torch.uint8, device=dev)
                a = _time(lambda: ours_ops.scaled_fp4_quant(kc, x, ks, gi, mask, n_ext, per8, False))
                b = _time(lambda: ref_ops.scaled_fp4_quant(kc, x, ks, gi, mask, n_ext, per8, False))
                rows.append(dict(kernel=f"nvfp4_kext_{ratio}", k=k, m=m, ours_us=round(a, 2), ref_us=round(b, 2),
                                 ours_gbs=round((2 * m * k + m * n_ext * 0.5625) / a / 1e3)))
            # ---- MXFP4 MEXT (row_pair, swizzled scales)
            mc = torch.empty(2 * m, k // 2, dtype=torch.uint8, device=dev)
            ms_ = torch.zeros(((2 * m + 127) // 128) * ((k // 32 + 3) // 4) * 512, dtype=torch.uint8, device=dev)
            a = _time(lambda: ours_ops.mxfp4_residue_quant(x, mc, ms_, None, 0, True, False, 0))
            b = _time(lambda: ref_ops.mxfp4_residue_quant(x, mc, ms_, None, 0, True, False, 0))
            rows.append(dict(kernel="mxfp4_mext", k=k, m=m, ours_us=round(a, 2), ref_us=round(b, 2),
                             ours_gbs=round((2 * m * k + 2 * m * k * 0.53125) / a / 1e3)))
    print()
    print(f"{'kernel':18s} {'K':>6s} {'M':>5s} {'ours us':>9s} {'ref us':>9s} {'ratio':>6s} {'ours GB/s':>10s}  plain order: ours / ref us")
    for r in rows:
        plain = f"  {r['ours_plain_us']:.2f} / {r['ref_plain_us']:.2f}" if "ours_plain_us" in r else ""
        print(f"{r['kernel']:18s} {r['k']:6d} {r['m']:5d} {r['ours_us']:9.2f} {r['ref_us']:9.2f} "
              f"{r['ours_us'] / r['ref_us']:6.2f} {r['ours_gbs']:10d}{plain}")
    out_dir = os.environ.get("RESINFER_B200_REPORT_DIR", "")
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "quantisers_vs_reference.json"), "w") as f:
            json.dump(rows, f, indent=1)
    slow = [r for r in rows if r["ours_us"] > 1.6 * r["ref_us"] + 0.3]
    assert not slow, slow
