"""GPU tests of the opaque linear ops and the registered linear modules (the calls a user makes)."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _setup(m, k, n, dev, per8=None):
    from resinfer_b200.quant import weight_prep
    x_np, w_np = O.make_activation(m, k, seed=2), O.make_weight(n, k, seed=3)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    w = torch.from_numpy(w_np).to(dev)
    idx = weight_prep.salient_indices_per8(k, per8, device=dev) if per8 else None
    prep = weight_prep.quantize_weight_nvfp4(w, idx)
    gs = float(np.abs(x_np).max()) / (6 * 448)
    gi = torch.tensor([1 / gs], dtype=torch.float32, device=dev)
    alpha = (prep["weight_global_scale"] * gs).float()
    return x_np, w_np, x, prep, gi, alpha, idx


@pytest.mark.parametrize("m", [1, 16, 128, 600])
def test_nvfp4_linear_ratio1_routes(cuda_device, m):
    """MEXT layer: fold route up to M = 512, K-concat route above; both equal the oracle contraction."""
    from resinfer_b200.quant.vllm_integration import residue_linear_op  # noqa: F401
    k, n = 512, 256
    x_np, w_np, x, prep, gi, alpha, _ = _setup(m, k, n, cuda_device)
    mask = torch.zeros(1, dtype=torch.uint8, device=cuda_device)
    y = torch.ops.residue.nvfp4_linear(x, prep["weight"], gi, prep["weight_scale"], prep["weight_scale_base"], mask,
                                       alpha, k, 0, 0, n, True, False, True)
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    codes, sf, _ = O.nvfp4_quant_mext(x_np, gi.cpu().numpy()[0], 1)
    a = O.dequant_operand(codes, sf, "nvfp4")
    wd = O.dequant_operand(prep["weight"].cpu().numpy(), prep["weight_scale"].cpu().numpy(), "nvfp4")
    ref = O.fp4_linear_reference(a[0::2] + a[1::2], wd, float(alpha.item()), False)
    assert rel_fro(y.detach().float().cpu().numpy(), ref) < 2.5e-3
    # and it beats plain W4A4 against the dense product
    y_plain = torch.ops.residue.nvfp4_linear(x, prep["weight"], gi, prep["weight_scale"], prep["weight_scale_base"],
                                             mask, alpha, k, 0, 0, n, False, False, False)
    dense = x_np.astype(np.float64) @ w_np.astype(np.float64).T
    assert rel_fro(y.detach().float().cpu().numpy(), dense) < rel_fro(y_plain.float().cpu().numpy(), dense)


@pytest.mark.parametrize("m,per8", [(16, 1), (200, 2), (300, 4)])
def test_nvfp4_linear_selective_routes(cuda_device, m, per8):
    """KEXT layer: decode-sized M folds on the base-K prefix of the extended weight (strided view),
    larger M runs the K-extended contraction."""
    from resinfer_b200.nvfp4.quant import indices_to_channel_masks
    from resinfer_b200.quant.vllm_integration import residue_linear_op  # noqa: F401
    k, n = 1024, 256
    x_np, w_np, x, prep, gi, alpha, idx = _setup(m, k, n, cuda_device, per8)
    mask = indices_to_channel_masks(idx, k)
    y = torch.ops.residue.nvfp4_linear(x, prep["weight"], gi, prep["weight_scale"], prep["weight_scale_base"], mask,
                                       alpha, k, idx.numel(), 0, n, True, False, False)
    wd = O.dequant_operand(prep["weight"].cpu().numpy(), prep["weight_scale"].cpu().numpy(), "nvfp4")
    if m <= 128:
        codes, sf, _ = O.nvfp4_quant_mext(x_np, gi.cpu().numpy()[0], 1)
        a = O.dequant_operand(codes, sf, "nvfp4")
        ref = O.fp4_linear_reference(a[0::2] + a[1::2], wd[:, :k], float(alpha.item()), False)
    else:
        codes, sf, _ = O.nvfp4_quant_kext(x_np, gi.cpu().numpy()[0], mask.cpu().numpy(), per8)
        ref = O.fp4_linear_reference(O.dequant_operand(codes, sf, "nvfp4"), wd, float(alpha.item()), False)
    assert rel_fro(y.detach().float().cpu().numpy(), ref) < 3e-3
    empty = torch.ops.residue.nvfp4_linear(x[:0], prep["weight"], gi, prep["weight_scale"], prep["weight_scale_base"],
                                           mask, alpha, k, idx.numel(), 0, n, True, False, False)
    assert empty.shape == (0, n)
    with pytest.raises(RuntimeError, match="Fold path"):
        torch.ops.residue.nvfp4_linear(x, prep["weight"], gi, prep["weight_scale"], prep["weight_scale_base"], mask,
                                       alpha, k, 0, 0, n, False, False, True)


@pytest.mark.parametrize("mode", ["standard", "selective", "mext_r1"])
def test_mxfp4_linear_modes(cuda_device, mode):
    from resinfer_b200.nvfp4.mxfp4 import prepare_indices
    from resinfer_b200.quant import mxfp4_linear, weight_prep  # noqa: F401
    m, k, n = 24, 512, 256
    x_np, w_np = O.make_activation(m, k, seed=4), O.make_weight(n, k, seed=5)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(cuda_device).reshape(2, 12, k)
    w = torch.from_numpy(w_np).to(cuda_device)
    sel = weight_prep.salient_indices_per8(k, 2, device=cuda_device) if mode == "selective" else None
    prep = weight_prep.quantize_weight_mxfp4(w, sel)
    if sel is not None:
        idx, masks = prepare_indices(sel.cpu(), k, cuda_device)
    else:
        idx = torch.zeros(0, dtype=torch.int32, device=cuda_device)
        masks = torch.zeros(0, dtype=torch.uint8, device=cuda_device)
    bias = torch.ones(n, dtype=torch.bfloat16, device=cuda_device)
    y = torch.ops.residue.mxfp4_linear(x, prep["weight"], prep["weight_scale"], idx, masks, mode, torch.bfloat16, bias)
    assert y.shape == (2, 12, n)
    dense = x_np.astype(np.float64) @ w_np.astype(np.float64).T + 1.0
    err = rel_fro(y.float().cpu().numpy().reshape(m, n), dense)
    assert err < {"standard": 0.2, "selective": 0.17, "mext_r1": 0.12}[mode]
    with pytest.raises(ValueError, match="unknown MXFP4 linear mode"):
        torch.ops.residue.mxfp4_linear(x, prep["weight"], prep["weight_scale"], idx, masks, "other", torch.bfloat16, None)


def test_registered_linear_modules(cuda_device):
    import resinfer_b200.quant.linear_impls  # noqa: F401
    from resinfer_b200.quant.linear_registry import LinearRegistry
    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 256, bias=True).to(cuda_device).to(torch.bfloat16)
    # 150 tokens: above the decode threshold (128), so the ratio-0.25 layer takes the masked K-extension
    # route while the ratio-1 layer stays on the fold route
    x = torch.randn(3, 50, 512, device=cuda_device).to(torch.bfloat16)
    dense = lin(x).detach().float()
    errs = {}
    for name, kw in (("NVFP4Linear", {}), ("ResidueLinear", {"ratio": 0.25}), ("ResidueLinear", {})):
        mod = LinearRegistry.get(name).from_linear(lin, input_amax=float(x.float().abs().max()), **kw)
        y = mod(x)
        assert y.shape == dense.shape
        errs[(name, kw.get("ratio", 1.0) if name == "ResidueLinear" else 0)] = rel_fro(y.detach().float().cpu().numpy(),
                                                                                      dense.cpu().numpy())
    assert errs[("ResidueLinear", 1.0)] < errs[("ResidueLinear", 0.25)] < errs[("NVFP4Linear", 0)] < 0.25
    with pytest.raises(NotImplementedError):
        LinearRegistry.get("ResidueSwapLinear").from_linear(lin)


def test_baseline_config0_mext_linear(cuda_device):
    """The CPU-runnable configuration of the baseline: x BF16 [16, 5120] (N(0,1), 1 % of channels x20),
    W BF16 [8192, 5120] (N(0, 0.02^2)), NVFP4 with FP32 global scales, y = deq(q(x)) deq(q(W))^T +
    deq(q(r)) deq(q(W))^T in FP32, BF16 out.  The op must equal the oracle's contraction of the same codes
    within BF16 rounding, and the torch-eager restatement of the reference's path within quantisation noise."""
    from resinfer_b200.quant.vllm_integration import residue_linear_op  # noqa: F401
    m, k, n = 16, 5120, 8192
    x_np, w_np, x, prep, gi, alpha, _ = _setup(m, k, n, cuda_device)
    mask = torch.zeros(1, dtype=torch.uint8, device=cuda_device)
    y = torch.ops.residue.nvfp4_linear(x, prep["weight"], gi, prep["weight_scale"], prep["weight_scale_base"], mask,
                                       alpha, k, 0, 0, n, True, False, True)
    got = y.detach().float().cpu().numpy()
    codes, sf, _ = O.nvfp4_quant_mext(x_np, gi.cpu().numpy()[0], 1)
    a = O.dequant_operand(codes, sf, "nvfp4")
    wd = O.dequant_operand(prep["weight"].cpu().numpy(), prep["weight_scale"].cpu().numpy(), "nvfp4")
    ref = O.fp4_linear_reference(a[0::2] + a[1::2], wd, float(alpha.item()), False)
    assert rel_fro(got, ref) < 2.5e-3
    eager = O.eager_residue_linear(torch.from_numpy(x_np).to(torch.bfloat16), torch.from_numpy(w_np).to(torch.bfloat16))
    assert rel_fro(got, eager.float().numpy()) < 2e-2
    dense = x_np.astype(np.float64) @ w_np.astype(np.float64).T
    assert rel_fro(got, dense) < 0.12
