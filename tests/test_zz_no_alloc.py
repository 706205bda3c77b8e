"""ri_fp4_gemm_static_scratch (the entry point that allocates nothing) against ri_fp4_gemm.

Collected last on purpose (file name): it must pass alone and after every other GPU test has used
the library.  Both entries run the same kernel with the same plan, so the two outputs must agree
within the tolerance the GEMM parity tests use; the call is made twice in a row because the second
call finds the shared scratch array as the first one left it."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-5       # relative Frobenius error, as in the GEMM parity tests
TOL_BF16 = 2.5e-3


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _case(m, n, k, dev, seed):
    from resinfer_b200 import nvfp4
    x_np, w_np = O.make_activation(m, k, seed=seed), O.make_weight(n, k, seed=seed + 1)
    gx = np.float32(np.abs(x_np).max() / (6 * 448))
    gw = np.float32(np.abs(w_np).max() / (6 * 448))
    wc, wsf = O.nvfp4_quant_plain(w_np, np.float32(1) / gw)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    gi = torch.tensor([1.0 / gx], dtype=torch.float32, device=dev)
    alpha = torch.tensor([float(gx) * float(gw)], dtype=torch.float32, device=dev)
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1)
    w = torch.from_numpy(np.ascontiguousarray(wc)).to(dev)
    w_sf = torch.from_numpy(np.ascontiguousarray(wsf)).to(dev)
    return codes, sf, w, w_sf, alpha


@pytest.mark.parametrize("m,n,k,splits", [(5, 1000, 4096, 0), (16, 256, 1024, 2), (64, 5120, 8192, 0),
                                         (128, 384, 1024, 1)])
def test_static_scratch_matches_workspace_entry(cuda_device, m, n, k, splits):
    from resinfer_b200 import _cabi, ops
    lib = _cabi.load()
    codes, sf, w, w_sf, alpha = _case(m, n, k, cuda_device, seed=11)
    if splits != 1:
        assert lib.ri_fp4_gemm_workspace_bytes(m, n, k, _cabi.FMT_NVFP4, _cabi.GEMM_ROW_PAIR, splits) > 0
    for dtype, tol in ((torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)):
        want = ops.fp4_gemm(codes, sf, w, w_sf, alpha, m=m, fmt="nvfp4", layout="row_pair", splits=splits,
                            out_dtype=dtype)
        for call in range(2):                                   # two calls in a row share the array
            got = torch.full((m, n), float("nan"), dtype=dtype, device=cuda_device)
            ops.fp4_gemm_static_scratch(codes, sf, w, w_sf, alpha, m=m, fmt="nvfp4", layout="row_pair",
                                        splits=splits, out=got)
            torch.cuda.synchronize()
            ops.check_status(cuda_device)
            assert torch.isfinite(got.float()).all(), (dtype, call)
            assert rel_fro(got.float().cpu().numpy(), want.float().cpu().numpy()) < tol, (dtype, call)


def test_static_scratch_rejects_oversized_problem(cuda_device):
    from resinfer_b200 import _cabi, ops
    lib = _cabi.load()
    # 4096 rows x 262144 columns: the ticket area alone is larger than the built-in array allows
    # together with the partial tiles; the check runs before any pointer is touched
    m, n, k = 4096, 1 << 21, 256
    need = lib.ri_fp4_gemm_workspace_bytes(m, n, k, _cabi.FMT_NVFP4, _cabi.GEMM_ROW_PAIR, 2)
    assert need > 20 * 1024 * 1024
    dummy = torch.zeros(256, dtype=torch.uint8, device=cuda_device)
    st = lib.ri_fp4_gemm_static_scratch(dummy.data_ptr(), k // 2, dummy.data_ptr(), 0, dummy.data_ptr(), k // 2,
                                        dummy.data_ptr(), 0, None, 0, dummy.data_ptr(), _cabi.DTYPE_BF16, n, m, n, k,
                                        _cabi.FMT_NVFP4, _cabi.GEMM_ROW_PAIR, 2, None, 0, None)
    assert st == _cabi.RI_ERR_ARG
    assert "built-in array" in _cabi.last_error()
    torch.cuda.synchronize()
    ops.check_status(cuda_device)
