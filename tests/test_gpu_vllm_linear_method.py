"""The vLLM linear method end to end on the GPU: weights created, loaded through the parameters' loaders, prepared by
``process_weights_after_loading`` and run by ``apply`` -- against the oracle's contraction of the very codes the
route produces (BF16 rounding tolerance) and against the dense BF16 product (quantisation error).  Modes:
K-extended layer with the decode fold switched on (fold route at M = 8, masked K extension at M = 200), a
``mext_r1`` layer (fold at every M) and a plain layer."""
import types

import numpy as np
import pytest
import torch

import oracle as O
from resinfer_b200.quant import kernel_metadata as KM
from resinfer_b200.quant import weight_prep
from resinfer_b200.quant.vllm_integration import env_contract

pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _build(name, mode, k, n, dev, monkeypatch):
    monkeypatch.setenv("RESIDUE_ENABLE_DECODE_MEXT", "1")
    env_contract.settings.cache_clear()
    from resinfer_b200.quant.vllm_integration.linear_method_v2 import ResidueNvFp4LinearMethodV2
    sel = {"extended_k": weight_prep.salient_indices_per8(k, 2), "mext_r1": torch.arange(k), "standard": None}[mode]
    layers = {} if sel is None else {name: sel}
    meta = KM.build_kernel_metadata(layers, residue_ratio=1.0 if mode == "mext_r1" else 0.25,
                                    in_features={name: k for name in layers})
    cfg = types.SimpleNamespace(group_size=16, is_checkpoint_nvfp4_serialized=True, _residue_metadata=meta)
    method = ResidueNvFp4LinearMethodV2(cfg, layer_prefix=name)
    layer = torch.nn.Module()
    layer.prefix = name
    method.create_weights(layer, k, [n], k, n, torch.bfloat16)
    layer.to(dev)
    w_np = O.make_weight(n, k, seed=31)
    w = torch.from_numpy(w_np)
    ext = sel if mode == "extended_k" else None
    packed = weight_prep.quantize_weight_nvfp4(w, ext)
    layer.weight.weight_loader(layer.weight, packed["weight"].to(dev))
    layer.weight_scale.weight_loader(layer.weight_scale, packed["weight_scale_raw"].view(torch.float8_e4m3fn).to(dev))
    layer.weight_scale_2.weight_loader(layer.weight_scale_2, packed["weight_global_scale"].reshape(1).to(dev))
    return method, layer, w_np, ext


@pytest.mark.parametrize("mode,m", [("extended_k", 8), ("extended_k", 200), ("mext_r1", 8), ("mext_r1", 300), ("standard", 40)])
def test_linear_method_against_the_oracle(cuda_device, monkeypatch, mode, m):
    dev = cuda_device
    k, n = 1024, 384
    name = "model.layers.0.self_attn.o_proj"
    method, layer, w_np, sel = _build(name, mode, k, n, dev, monkeypatch)
    x_np = O.make_activation(m, k, seed=7)
    gs = float(np.abs(x_np).max()) / (6 * 448)
    layer.input_scale.weight_loader(layer.input_scale, torch.tensor([gs], device=dev))
    if sel is not None:
        layer.input_quantizer._salient_indices = sel.to(dev)
    method.process_weights_after_loading(layer)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    bias = torch.full((n,), 0.25, dtype=torch.bfloat16, device=dev)
    y = method.apply(layer, x.view(1, m, k), bias)
    torch.cuda.synchronize()
    from resinfer_b200 import ops
    ops.check_status(dev)
    assert y.shape == (1, m, n) and y.dtype == torch.bfloat16
    got = (y.float() - 0.25).view(m, n).cpu().numpy()
    alpha = float(layer.alpha.item())
    wd = O.dequant_operand(layer.weight.cpu().numpy(), layer.weight_scale.view(torch.uint8).reshape(-1).cpu().numpy(), "nvfp4")
    gi = np.float32(1 / gs)
    fold = mode == "mext_r1" or m <= 128                          # the op's routing (decode fold up to 128 tokens)
    if mode == "standard" and not fold:
        raise AssertionError("test shape must stay on the fold route")
    if fold:
        codes, sf, _ = O.nvfp4_quant_mext(x_np, gi, 1)
        a = O.dequant_operand(codes, sf, "nvfp4")
        ref = O.fp4_linear_reference(a[0::2] + a[1::2], wd[:, :k], alpha, False)
    else:
        codes, sf = O.nvfp4_quant_kext(x_np, gi, layer.channel_mask.cpu().numpy(), 2)[:2]
        ref = O.fp4_linear_reference(O.dequant_operand(codes, sf, "nvfp4"), wd, alpha, False)
    assert rel_fro(got, ref) < 6e-3                               # BF16 output (+ BF16 bias add), approximate reciprocals
    assert rel_fro(got, x_np.astype(np.float64) @ w_np.astype(np.float64).T) < 0.15
    env_contract.settings.cache_clear()


@pytest.mark.parametrize("mode,m", [("selective", 40), ("mext_r1", 8), ("standard", 130)])
def test_mxfp4_linear_method_against_the_oracle(cuda_device, mode, m):
    from resinfer_b200.quant.vllm_integration.linear_method_mxfp4 import ResidueMxfp4LinearMethod
    dev = cuda_device
    k, n = 1024, 384
    sel = {"selective": weight_prep.salient_indices_per8(k, 2), "mext_r1": torch.arange(k), "standard": None}[mode]
    rec = {} if sel is None else {"runtime_mode": "mext_r1" if mode == "mext_r1" else "extended_k",
                                  "num_salient": sel.numel(), "salient_indices": sel.tolist()}
    method = ResidueMxfp4LinearMethod(rec)
    layer = torch.nn.Module()
    method.create_weights(layer, k, [n], k, n, torch.bfloat16)
    layer.to(dev)
    w_np = O.make_weight(n, k, seed=41)
    packed = weight_prep.quantize_weight_mxfp4(torch.from_numpy(w_np), sel if mode == "selective" else None)
    assert layer.weight.shape == packed["weight"].shape
    layer.weight.weight_loader(layer.weight, packed["weight"].to(dev))
    layer.weight_scale.weight_loader(layer.weight_scale, packed["weight_scale_raw"].to(dev))
    method.process_weights_after_loading(layer)
    assert layer._mxfp4_prepared and not isinstance(layer.weight_scale, torch.nn.Parameter)
    assert torch.equal(layer.weight_scale.cpu(), packed["weight_scale"])                    # swizzled after loading
    x_np = O.make_activation(m, k, seed=8)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    y = method.apply(layer, x.view(1, m, k), None)
    torch.cuda.synchronize()
    from resinfer_b200 import ops
    ops.check_status(dev)
    assert y.shape == (1, m, n) and y.dtype == torch.bfloat16
    got = y.float().view(m, n).cpu().numpy()
    wd = O.dequant_operand(packed["weight"].numpy(), packed["weight_scale"].numpy(), "mxfp4")
    if mode == "mext_r1":
        codes, sf = O.mxfp4_quant_mext(x_np)[:2]
        a = O.dequant_operand(codes, sf, "mxfp4")
        ref = O.fp4_linear_reference(a[0::2] + a[1::2], wd, 1.0, False)
    elif mode == "selective":
        codes, sf = O.mxfp4_quant_selective(x_np, layer.salient_masks.cpu().numpy(), 2, kp=wd.shape[1])[:2]
        ref = O.fp4_linear_reference(O.dequant_operand(codes, sf, "mxfp4"), wd, 1.0, False)
    else:
        codes, sf = O.mxfp4_quant_plain(x_np)[:2]
        ref = O.fp4_linear_reference(O.dequant_operand(codes, sf, "mxfp4"), wd, 1.0, False)
    assert rel_fro(got, ref) < 5e-3
    # quantisation error against the dense product: plain W4A4 MXFP4 (no residue) is the coarsest of the three
    assert rel_fro(got, x_np.astype(np.float64) @ w_np.astype(np.float64).T) < (0.25 if mode == "standard" else 0.2)
    # NaN scale codes are refused
    bad = torch.nn.Module()
    m2 = ResidueMxfp4LinearMethod(rec)
    m2.create_weights(bad, k, [n], k, n, torch.bfloat16)
    bad.to(dev)
    with pytest.raises(ValueError, match="incomplete packed MXFP4"):                        # nothing loaded yet
        m2.process_weights_after_loading(bad)
    bad.weight.weight_loader(bad.weight, packed["weight"].to(dev))
    bad.weight_scale.weight_loader(bad.weight_scale, torch.full_like(packed["weight_scale_raw"], 255).to(dev))
    with pytest.raises(ValueError, match="NaN E8M0"):
        m2.process_weights_after_loading(bad)
