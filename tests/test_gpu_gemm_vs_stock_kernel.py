"""The FP4 GEMM against a second, independent BF16 kernel on the SAME codes and scales: the stock
block-scaled GEMM of the FlashInfer library (``flashinfer.mm_fp4``, cuDNN backend: no JIT build), called
the way the reference calls it on its prefill route (ShawRong/ResInfer
quant/vllm_integration/residue_linear_op.py:46-70: row-pair activation codes as 2M rows, weights and
128x4-swizzled scales transposed, then ``y[0::2] + y[1::2]``).

FlashInfer is a comparison kernel here and nothing more: it is imported by this test only.

Tolerances.  Two BF16 kernels that accumulate the same products in FP32 differ only where the last FP32
bits flip a BF16 rounding: the plain GEMM over the 2M rows must agree within 1e-3 relative Frobenius
(measured: bit-identical).  The reference's two-GEMM route rounds base and residue products to BF16
separately and adds them in BF16, this library's fold adds them in FP32 and rounds once, so those two differ
by BF16 rounding of the larger term (about 2.9e-3 measured); the bound for that comparison is 4e-3.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_SAME_CONTRACTION = 1e-3
TOL_TWO_GEMM_ROUTE = 4e-3


def rel_fro(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.fixture(scope="module")
def mm_fp4():
    try:
        from flashinfer import mm_fp4 as fn
    except Exception as e:                                   # the comparison kernel is optional equipment
        pytest.skip(f"flashinfer.mm_fp4 not importable: {type(e).__name__}: {e}")
    return fn


@pytest.mark.parametrize("m,k,n", [(64, 5120, 10240), (16, 25600, 5120), (128, 8192, 5120), (1, 5120, 51200)])
def test_nvfp4_against_flashinfer_mm_fp4(cuda_device, mm_fp4, m, k, n):
    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.quant import weight_prep
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(m + n)
    x = torch.randn(m, k, generator=g, device=dev, dtype=torch.float32)
    x[:, torch.randperm(k, generator=g, device=dev)[: k // 100]] *= 20.0
    x = x.to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    prep = weight_prep.quantize_weight_nvfp4(w)
    del w
    gs = float(x.float().abs().max()) / (6 * 448)
    gi = torch.tensor([1 / gs], dtype=torch.float32, device=dev)
    alpha = (prep["weight_global_scale"] * gs).float().reshape(1)
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1)          # row_pair: [2M, K/2]
    two_m = codes.shape[0]
    x_sf = sf.view(torch.float8_e4m3fn).view(((two_m + 127) // 128) * 128, (k // 64) * 4)
    w_sf = prep["weight_scale"].view(torch.float8_e4m3fn).view(((n + 127) // 128) * 128, (k // 64) * 4)
    try:
        stock = mm_fp4(codes, prep["weight"].T, x_sf, w_sf.T, alpha, torch.bfloat16, backend="cudnn")
    except Exception as e:
        pytest.skip(f"flashinfer.mm_fp4(backend='cudnn') does not run here: {type(e).__name__}: {str(e)[:200]}")
    ours_rows = ops.fp4_gemm(codes, sf, prep["weight"], prep["weight_scale"], alpha, m=two_m, fmt="nvfp4", layout="plain")
    ours_fold = ops.fp4_gemm(codes, sf, prep["weight"], prep["weight_scale"], alpha, m=m, fmt="nvfp4", layout="row_pair")
    torch.cuda.synchronize()
    ops.check_status(dev)
    assert stock.shape == ours_rows.shape
    assert rel_fro(ours_rows, stock) < TOL_SAME_CONTRACTION
    assert rel_fro(ours_fold, stock[0::2] + stock[1::2]) < TOL_TWO_GEMM_ROUTE
    # the fold is the closer of the two to the unrounded sum of the stock kernel's rows
    assert rel_fro(ours_fold, stock[0::2].float() + stock[1::2].float()) < TOL_TWO_GEMM_ROUTE
