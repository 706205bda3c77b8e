"""GPU parity of the tcgen05 block-scaled GEMM against the FP32 product of the dequantised operands
(the oracle): FP32 output within 2e-5 relative Frobenius error (accumulation order only), BF16 output
within the BF16 rounding of the result."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-5       # relative Frobenius, unrounded output vs float64-accumulated oracle
TOL_BF16 = 2.5e-3    # BF16 output: rounding to 8 significant bits alone gives about 1.6e-3


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _nvfp4_case(m, n, k, dev, seed=1):
    from resinfer_b200 import nvfp4
    x_np, w_np = O.make_activation(m, k, seed=seed), O.make_weight(n, k, seed=seed + 1)
    gx = np.float32(np.abs(x_np).max() / (6 * 448))
    gw = np.float32(np.abs(w_np).max() / (6 * 448))
    wc, wsf = O.nvfp4_quant_plain(w_np, np.float32(1) / gw)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    gi = torch.tensor([1.0 / gx], dtype=torch.float32, device=dev)
    alpha = torch.tensor([float(gx) * float(gw)], dtype=torch.float32, device=dev)
    return x_np, w_np, x, gi, alpha, wc, wsf


@pytest.mark.parametrize("m,n,k,splits", [(1, 128, 256, 1), (16, 256, 512, 1), (16, 256, 1024, 2), (128, 384, 1024, 1),
                                         (100, 200, 2048, 4), (300, 256, 512, 1), (5, 1000, 4096, 0),
                                         (64, 5120, 8192, 0),
                                         # an odd number of 256-element K tiles: the last 512-element stage is half empty
                                         (16, 256, 1280, 1), (8, 384, 2304, 0), (48, 640, 3328, 2)])
def test_nvfp4_fold_layouts(cuda_device, m, n, k, splits):
    from resinfer_b200 import nvfp4, ops
    x_np, w_np, x, gi, alpha, wc, wsf = _nvfp4_case(m, n, k, cuda_device)
    w_deq = O.dequant_operand(wc, wsf, "nvfp4")
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1)
    a = O.dequant_operand(codes.cpu().numpy(), sf.cpu().numpy(), "nvfp4")
    ref = O.fp4_linear_reference(a[0::2] + a[1::2], w_deq, float(alpha.item()), round_bf16=False)
    outs = {}
    for lname, lay in (("row_pair", 1), ("concat_k", 3)):
        c, s = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=lay)
        y32 = ops.fp4_gemm(c, s, _t(wc, cuda_device), _t(wsf, cuda_device), alpha, m=m, fmt="nvfp4", layout=lname,
                           splits=splits, out_dtype=torch.float32)
        y16 = ops.fp4_gemm(c, s, _t(wc, cuda_device), _t(wsf, cuda_device), alpha, m=m, fmt="nvfp4", layout=lname,
                           splits=splits)
        torch.cuda.synchronize()
        ops.check_status(cuda_device)
        assert rel_fro(y32.cpu().numpy(), ref) < TOL_F32, lname
        assert rel_fro(y16.float().cpu().numpy(), ref) < TOL_BF16, lname
        assert torch.equal(y16, y32.to(torch.bfloat16))         # BF16 output = rounded FP32 output
        outs[lname] = y32
    # same contraction through both layouts
    assert rel_fro(outs["row_pair"].cpu().numpy(), outs["concat_k"].cpu().numpy()) < TOL_F32


@pytest.mark.parametrize("m,n,k,per8", [(16, 256, 512, 2), (128, 384, 1024, 1), (300, 256, 1024, 4), (16, 512, 5120, 1)])
def test_nvfp4_kext_plain_layout_with_partial_k_tile(cuda_device, m, n, k, per8):
    """KEXT: K + S is a multiple of 64 but not always of 256 (5120 * 1.125 = 5760)."""
    from resinfer_b200 import nvfp4, ops
    x_np, w_np, x, gi, alpha, _, _ = _nvfp4_case(m, n, k, cuda_device, seed=3)
    mask_np = O.make_kext_mask(k, per8)
    sel = O.mask_to_indices(mask_np)
    gw = np.float32(np.abs(w_np).max() / (6 * 448))
    wc, wsf = O.nvfp4_quant_plain(np.concatenate([w_np, w_np[:, sel]], axis=1), np.float32(1) / gw)
    codes, sf = nvfp4.scaled_fp4_quant_with_mask(x, gi, _t(mask_np, cuda_device), sel.size)
    y = ops.fp4_gemm(codes, sf, _t(wc, cuda_device), _t(wsf, cuda_device), alpha, m=m, fmt="nvfp4", layout="plain",
                     out_dtype=torch.float32)
    torch.cuda.synchronize()
    ops.check_status(cuda_device)
    a = O.dequant_operand(codes.cpu().numpy(), sf.cpu().numpy(), "nvfp4")
    ref = O.fp4_linear_reference(a, O.dequant_operand(wc, wsf, "nvfp4"), float(alpha.item()), round_bf16=False)
    assert rel_fro(y.cpu().numpy(), ref) < TOL_F32


@pytest.mark.parametrize("m,n,k,splits", [(1, 128, 256, 1), (16, 256, 1024, 2), (100, 224, 2048, 4), (130, 256, 640, 1),
                                         (16, 256, 1408, 1)])          # 5.5 K tiles of 256: half a 512-element stage at the end
def test_mxfp4_gemms(cuda_device, m, n, k, splits):
    from resinfer_b200 import ops
    from resinfer_b200.nvfp4 import mxfp4 as mx
    x_np, w_np = O.make_activation(m, k, seed=5), O.make_weight(n, k, seed=6)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(cuda_device)
    wc, wsf = O.mxfp4_quant_plain(w_np)
    w_deq = O.dequant_operand(wc, wsf, "mxfp4")
    codes, sf = mx.quantize_mext(x)
    y = ops.fp4_gemm(codes, sf, _t(wc, cuda_device), _t(wsf, cuda_device), None, m=m, fmt="mxfp4", layout="row_pair",
                     splits=splits, out_dtype=torch.float32)
    a = O.dequant_operand(codes.cpu().numpy(), sf.cpu().numpy(), "mxfp4")
    assert rel_fro(y.cpu().numpy(), O.fp4_linear_reference(a[0::2] + a[1::2], w_deq, 1.0, False)) < TOL_F32
    # reference-named entry points: fold_gemm / gemm, BF16 output
    yb = mx.fold_gemm(codes, _t(wc, cuda_device), sf, _t(wsf, cuda_device))
    assert torch.equal(yb, y.to(torch.bfloat16)) or rel_fro(yb.float().cpu().numpy(), y.cpu().numpy()) < TOL_BF16
    pc, ps = mx.quantize(x)
    yp = mx.gemm(pc, _t(wc, cuda_device), ps, _t(wsf, cuda_device), out_dtype=torch.float16)
    ap = O.dequant_operand(pc.cpu().numpy(), ps.cpu().numpy(), "mxfp4")
    assert rel_fro(yp.float().cpu().numpy(), O.fp4_linear_reference(ap, w_deq, 1.0, False)) < 1e-3
    torch.cuda.synchronize()
    ops.check_status(cuda_device)


def test_fold_host_api_dual_alpha_and_strided_weight(cuda_device):
    from resinfer_b200 import nvfp4
    from resinfer_b200.nvfp4.cute_fold.host import kext_kloop_gemm_sm100, mext_fold_gemm
    m, n, k = 24, 256, 512
    x_np, w_np, x, gi, alpha, wc, wsf = _nvfp4_case(m, n, k, cuda_device, seed=7)
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1)
    a = O.dequant_operand(codes.cpu().numpy(), sf.cpu().numpy(), "nvfp4")
    w_deq = O.dequant_operand(wc, wsf, "nvfp4")
    al = float(alpha.item())
    y = mext_fold_gemm(_t(wc, cuda_device), codes, _t(wsf, cuda_device), sf, alpha, alpha_res=alpha * 0.5)
    ref = O.fp4_linear_reference(a[0::2] + 0.5 * a[1::2], w_deq, al, False)
    assert rel_fro(y.float().cpu().numpy(), ref) < TOL_BF16
    # K-extended weight buffer, base-K prefix used as a strided view (decode MExt on a KEXT layer)
    wide = torch.zeros(n, k // 2 + 64, dtype=torch.uint8, device=cuda_device)
    wide[:, :k // 2] = _t(wc, cuda_device)
    y2 = mext_fold_gemm(wide[:, :k // 2], codes, _t(wsf, cuda_device), sf, alpha)
    assert rel_fro(y2.float().cpu().numpy(), O.fp4_linear_reference(a[0::2] + a[1::2], w_deq, al, False)) < TOL_BF16
    ck, sk = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=3)
    y3 = kext_kloop_gemm_sm100(_t(wc, cuda_device), ck, _t(wsf, cuda_device), sk, alpha)
    assert rel_fro(y3.float().cpu().numpy(), y2.float().cpu().numpy()) < 2e-3
    with pytest.raises(ValueError, match="compact"):
        mext_fold_gemm(_t(wc, cuda_device), codes[::2], _t(wsf, cuda_device), sf, alpha)
    with pytest.raises(ValueError, match="SM100"):
        mext_fold_gemm(_t(wc, cuda_device), codes, _t(wsf, cuda_device), sf, alpha, kernel_arch="sm103")


def test_gemm_properties_at_baseline_size(cuda_device):
    """Size-independent properties on a benchmarked shape (qkv 5120 -> 10240, M = 128): split-K invariance,
    row independence (a token's output does not depend on the other tokens) and scaling in alpha."""
    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.quant import weight_prep
    m, k, n = 128, 5120, 10240
    g = torch.Generator(device=cuda_device).manual_seed(0)
    x = torch.randn(m, k, generator=g, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device=cuda_device) * 0.02).to(torch.bfloat16)
    prep = weight_prep.quantize_weight_nvfp4(w)
    gs = float(x.float().abs().max()) / (6 * 448)
    gi = torch.tensor([1 / gs], dtype=torch.float32, device=cuda_device)
    alpha = (prep["weight_global_scale"] * gs).float()
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1)
    run = lambda c, s, mm, **kw: ops.fp4_gemm(c, s, prep["weight"], prep["weight_scale"], kw.pop("alpha", alpha), m=mm,
                                              fmt="nvfp4", layout="row_pair", out_dtype=torch.float32, **kw)
    y1 = run(codes, sf, m, splits=1)
    y4 = run(codes, sf, m, splits=4)
    assert rel_fro(y4.cpu().numpy(), y1.cpu().numpy()) < TOL_F32
    assert torch.equal(run(codes, sf, m, splits=4), y4)                       # deterministic
    c8, s8 = nvfp4.scaled_fp4_quant_mext_r1(x[:8].contiguous(), gi, layout_mode=1)
    y8 = run(c8, s8, 8, splits=0)
    assert rel_fro(y8.cpu().numpy(), y1[:8].cpu().numpy()) < TOL_F32
    y2a = run(codes, sf, m, splits=1, alpha=alpha * 2)
    assert torch.allclose(y2a, 2 * y1, rtol=1e-6, atol=0)
    # against the dense BF16 product: W4A4 + residue stays within quantisation error
    dense = x.float() @ w.float().t()
    assert rel_fro(y1.cpu().numpy(), dense.cpu().numpy()) < 0.12
    torch.cuda.synchronize()
    ops.check_status(cuda_device)


def test_gemm_rejects_bad_arguments(cuda_device):
    from resinfer_b200 import ops
    a = torch.zeros(4, 100, dtype=torch.uint8, device=cuda_device)
    w = torch.zeros(128, 100, dtype=torch.uint8, device=cuda_device)
    sf = torch.zeros(4096, dtype=torch.uint8, device=cuda_device)
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.fp4_gemm(a, sf, w, sf, None, m=4, fmt="nvfp4", layout="plain")
    a = torch.zeros(4, 128, dtype=torch.uint8, device=cuda_device)
    w = torch.zeros(128, 128, dtype=torch.uint8, device=cuda_device)
    with pytest.raises(RuntimeError, match="scale buffer"):
        ops.fp4_gemm(a, sf[:16], w, sf, None, m=4, fmt="nvfp4", layout="plain")
    with pytest.raises(RuntimeError, match="MXFP4 has no global scale"):
        ops.fp4_gemm(a, sf, w, sf, torch.ones(1, device=cuda_device), m=4, fmt="mxfp4", layout="plain")
    assert ops.fp4_gemm(a[:0], sf, w, sf, None, m=0, fmt="nvfp4", layout="plain").shape == (0, 128)


@pytest.mark.parametrize("fmt,m,n,k,layout", [("nvfp4", 128, 384, 1024, "row_pair"), ("nvfp4", 300, 512, 512, "plain"),
                                              ("nvfp4", 256, 1000, 2048, "concat_k"), ("mxfp4", 130, 384, 640, "row_pair"),
                                              ("nvfp4", 520, 2560, 5120, "row_pair")])
def test_two_cta_tiles_against_one_cta_tiles(cuda_device, fmt, m, n, k, layout):
    """Plans with 256 accumulator columns can run as pairs of CTAs on 256-row weight tiles
    (tcgen05.mma.cta_group::2, ``splits=-2``).  Same products in the same K order as the one-CTA tiles
    (``splits=1``): the FP32 outputs must agree to rounding noise, and both with the oracle.  Shapes cover an
    odd number of 128-row tiles (the last pair is half empty), a ragged last tile and several token tiles."""
    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.nvfp4 import mxfp4 as mx
    dev = cuda_device
    x_np, w_np = O.make_activation(m, k, seed=11), O.make_weight(n, k, seed=12)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    if fmt == "nvfp4":
        gx = np.float32(np.abs(x_np).max() / (6 * 448))
        gw = np.float32(np.abs(w_np).max() / (6 * 448))
        wc, wsf = O.nvfp4_quant_plain(w_np, np.float32(1) / gw)
        gi = torch.tensor([1.0 / gx], dtype=torch.float32, device=dev)
        alpha = torch.tensor([float(gx) * float(gw)], dtype=torch.float32, device=dev)
        if layout == "plain":
            codes = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
            sf = torch.zeros(((m + 127) // 128) * ((k + 63) // 64) * 512, dtype=torch.uint8, device=dev)
            torch.ops.nvfp4.scaled_fp4_quant_mext_r1(codes, x, sf, gi, 0, 5, True)
        else:
            codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1 if layout == "row_pair" else 3)
    else:
        wc, wsf = O.mxfp4_quant_plain(w_np)
        codes, sf = mx.quantize_mext(x)
        alpha = None
    run = lambda s: ops.fp4_gemm(codes, sf, _t(wc, dev), _t(wsf, dev), alpha, m=m, fmt=fmt, layout=layout, splits=s,   # noqa: E731
                                 out_dtype=torch.float32)
    y_pair, y_one = run(-2), run(1)
    torch.cuda.synchronize()
    ops.check_status(dev)
    assert rel_fro(y_pair.cpu().numpy(), y_one.cpu().numpy()) < 1e-6
    a = O.dequant_operand(codes.cpu().numpy(), sf.cpu().numpy(), fmt)
    if layout == "row_pair":
        a = a[0::2] + a[1::2]
    elif layout == "concat_k":
        a = a[:, :k] + a[:, k:]
    ref = O.fp4_linear_reference(a, O.dequant_operand(wc, wsf, fmt), 1.0 if alpha is None else float(alpha.item()), False)
    assert rel_fro(y_pair.cpu().numpy(), ref) < TOL_F32
    yb = ops.fp4_gemm(codes, sf, _t(wc, dev), _t(wsf, dev), alpha, m=m, fmt=fmt, layout=layout, splits=-2)
    assert torch.equal(yb, y_pair.to(torch.bfloat16))
