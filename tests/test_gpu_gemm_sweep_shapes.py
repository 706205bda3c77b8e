"""GPU parity of the FP4 GEMM at the shapes and plans the benchmark runs: the four Qwen3-32B-shaped
projections (qkv 5120->10240, o 8192->5120, gate_up 5120->51200, down 25600->5120) at M in {1, 16, 128},
NVFP4 and MXFP4 MEXT (row_pair fold) with the planner's own choice of work split (``splits=0``), plus
KEXT (ratio 0.125, plain layout over K + S) and the ratio-1 K-concat route at M = 1024 on qkv.

Two independent checkers per case:
  * the numpy oracle: the float64-accumulated product of the dequantised operands on a sample of at least
    512 weight rows (first and last tile, every 128-row tile boundary of a strided subset, seeded random
    rows) times all tokens;
  * a float64 matmul in torch over the whole output (a second dequantiser written with torch look-ups),
    so that every output tile of every CTA range is compared with something.
Tolerances: FP32 output <= 2e-5 relative Frobenius (accumulation order only); BF16 output <= 2.5e-3
(rounding to 8 significant bits alone is about 1.6e-3) and bit-equal to the rounded FP32 output.
"""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-5
TOL_BF16 = 2.5e-3
SHAPES = {"qkv": (5120, 10240), "o": (8192, 5120), "gate_up": (5120, 51200), "down": (25600, 5120)}
E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def rel_fro_t(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def unswizzle(buf: torch.Tensor, rows: int, groups: int) -> torch.Tensor:
    """128x4-swizzled scale bytes -> [rows, groups] (inverse of weight_prep.swizzle_scales_any)."""
    rt, kt = (rows + 127) // 128, (groups + 3) // 4
    lin = buf.reshape(-1)[: rt * kt * 512].reshape(rt, kt, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(rt * 128, kt * 4)
    return lin[:rows, :groups]


def dequant_torch(codes: torch.Tensor, sf_lin: torch.Tensor, fmt: str) -> torch.Tensor:
    """uint8 codes [R, K/2] + linear scale bytes [R, K/vec] -> float64 [R, K] (torch look-ups)."""
    lut = torch.tensor(E2M1 + tuple(-v for v in E2M1), dtype=torch.float64, device=codes.device)
    lo, hi = codes & 0xF, codes >> 4
    vals = torch.stack([lut[lo.long()], lut[hi.long()]], dim=-1).reshape(codes.shape[0], -1)
    if fmt == "nvfp4":
        sc = sf_lin.contiguous().view(torch.float8_e4m3fn).double()
        vec = 16
    else:
        sc = torch.where(sf_lin == 0, torch.zeros((), dtype=torch.float64, device=codes.device),
                         torch.exp2(sf_lin.double() - 127.0))
        vec = 32
    return (vals.reshape(codes.shape[0], -1, vec) * sc[..., None]).reshape(codes.shape[0], -1)


def sample_rows(n: int, seed: int = 0) -> np.ndarray:
    tiles = n // 128
    rows = set(range(128)) | set(range(n - 128, n))
    for t in range(1, tiles, max(1, tiles // 64)):
        rows |= {128 * t - 1, 128 * t}
    rng = np.random.default_rng(seed)
    rows |= set(int(r) for r in rng.integers(0, n, size=320))
    return np.array(sorted(rows), dtype=np.int64)


def make_x(m, k, dev, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(m, k, generator=g, device=dev, dtype=torch.float32)
    x[:, torch.randperm(k, generator=g, device=dev)[: max(1, k // 100)]] *= 20.0
    return x.to(torch.bfloat16)


_WEIGHTS = {}


def prepared_weight(name, fmt, dev, idx=None, tag=""):
    """Prequantised weight of a projection (cached per session: the quantisation is torch code)."""
    from resinfer_b200.quant import weight_prep
    key = (name, fmt, tag)
    if key not in _WEIGHTS:
        k, n = SHAPES[name]
        g = torch.Generator(device=dev).manual_seed(11)
        w = (torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        prep = (weight_prep.quantize_weight_mxfp4 if fmt == "mxfp4" else weight_prep.quantize_weight_nvfp4)(w, idx)
        _WEIGHTS.clear()                                   # one prepared weight at a time is enough
        _WEIGHTS[key] = prep
    return _WEIGHTS[key]


def check_against_both(y32, y16, a_deq, prep, fmt, alpha, dev):
    """a_deq: float64 [M, Kx] effective activation (residue already folded where the layout folds)."""
    wc, wsf = prep["weight"], prep["weight_scale"]
    n, kx = wc.shape[0], wc.shape[1] * 2
    vec = 16 if fmt == "nvfp4" else 32
    sf_lin = unswizzle(wsf, n, kx // vec)
    # ---- whole output against torch float64
    ref_full = (a_deq @ dequant_torch(wc, sf_lin, fmt).t()) * alpha
    assert rel_fro_t(y32, ref_full) < TOL_F32
    assert rel_fro_t(y16.float(), ref_full) < TOL_BF16
    assert torch.equal(y16, y32.to(torch.bfloat16))
    # worst single output column against the typical column norm (a weight row that went wrong would
    # hide in the Frobenius norm of 51200 columns)
    col_err = (y32.double() - ref_full).norm(dim=0) / (ref_full.norm() / ref_full.shape[1] ** 0.5)
    assert float(col_err.max()) < 1e-3
    # ---- sampled weight rows against the numpy oracle
    rows = sample_rows(n)
    assert rows.size >= 512
    r_t = torch.from_numpy(rows).to(dev)
    w_rows = (O.nvfp4_dequant if fmt == "nvfp4" else O.mxfp4_dequant)(wc[r_t].cpu().numpy(), sf_lin[r_t].cpu().numpy())
    ref = O.fp4_linear_reference(a_deq.cpu().numpy(), w_rows, alpha, round_bf16=False)
    got = y32[:, r_t].cpu().numpy().astype(np.float64)
    assert float(np.linalg.norm(got - ref) / np.linalg.norm(ref)) < TOL_F32


@pytest.mark.parametrize("m", [1, 16, 128])
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_mext_fold_at_sweep_shapes(cuda_device, name, fmt, m):
    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.nvfp4 import mxfp4 as mx
    dev = cuda_device
    k, n = SHAPES[name]
    prep = prepared_weight(name, fmt, dev)
    x = make_x(m, k, dev)
    if fmt == "nvfp4":
        gs = float(x.float().abs().max()) / (6 * 448)
        gi = torch.tensor([1 / gs], dtype=torch.float32, device=dev)
        alpha_t = (prep["weight_global_scale"] * gs).float().reshape(1)
        codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1)
        alpha = float(alpha_t.item())
    else:
        codes, sf = mx.quantize_mext(x)
        alpha_t, alpha = None, 1.0
    run = lambda dt: ops.fp4_gemm(codes, sf, prep["weight"], prep["weight_scale"], alpha_t, m=m, fmt=fmt,   # noqa: E731
                                  layout="row_pair", splits=0, out_dtype=dt)
    y32, y16 = run(torch.float32), run(torch.bfloat16)
    torch.cuda.synchronize()
    ops.check_status(dev)
    vec = 16 if fmt == "nvfp4" else 32
    a = dequant_torch(codes, unswizzle(sf, 2 * m, k // vec), fmt)
    # the torch dequantiser of the activation agrees with the oracle's
    a_np = O.dequant_operand(codes.cpu().numpy(), sf.cpu().numpy(), fmt)
    assert np.array_equal(a.cpu().numpy().astype(np.float32), a_np)
    check_against_both(y32, y16, a[0::2] + a[1::2], prep, fmt, alpha, dev)


@pytest.mark.parametrize("route", ["kext_0.125", "concat_k"])
def test_kext_and_kconcat_at_m1024_on_qkv(cuda_device, route):
    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.nvfp4.quant import indices_to_channel_masks
    from resinfer_b200.quant import weight_prep
    dev = cuda_device
    m, (k, n) = 1024, SHAPES["qkv"]
    x = make_x(m, k, dev, seed=4)
    gs = float(x.float().abs().max()) / (6 * 448)
    gi = torch.tensor([1 / gs], dtype=torch.float32, device=dev)
    if route == "concat_k":
        prep = prepared_weight("qkv", "nvfp4", dev)
        codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=3)          # [M, K] bytes = base | residue
        a2 = dequant_torch(codes, unswizzle(sf, m, 2 * k // 16), "nvfp4")
        a = a2[:, :k] + a2[:, k:]
        layout = "concat_k"
    else:
        idx = weight_prep.salient_indices_per8(k, 1, device=dev)
        prep = prepared_weight("qkv", "nvfp4", dev, idx, tag="kext1")
        mask = indices_to_channel_masks(idx, k)
        codes, sf = nvfp4.scaled_fp4_quant_with_mask(x, gi, mask, idx.numel(), use_swapped_residue=False)
        a = dequant_torch(codes, unswizzle(sf, m, (k + idx.numel()) // 16), "nvfp4")
        layout = "plain"
    alpha_t = (prep["weight_global_scale"] * gs).float().reshape(1)
    run = lambda dt: ops.fp4_gemm(codes, sf, prep["weight"], prep["weight_scale"], alpha_t, m=m, fmt="nvfp4",   # noqa: E731
                                  layout=layout, splits=0, out_dtype=dt)
    y32, y16 = run(torch.float32), run(torch.bfloat16)
    torch.cuda.synchronize()
    ops.check_status(dev)
    check_against_both(y32, y16, a, prep, "nvfp4", float(alpha_t.item()), dev)
