"""The vLLM linear method of the residue NVFP4 path on CPU: weight creation (extended K, row-parallel shard plan and
loader interleave), the state built after loading (scales, masks, base-K scale buffer, modes) and the arguments
``apply`` hands to ``residue::nvfp4_linear`` -- the behaviour of the reference's
quant/vllm_integration/linear_method_v2.py:105-618, driven with plain modules in place of vLLM layers."""
import types

import pytest
import torch

from resinfer_b200.quant import kernel_metadata as KM
from resinfer_b200.quant import weight_prep
from resinfer_b200.quant.vllm_integration import env_contract


@pytest.fixture()
def method_cls(monkeypatch):
    for k in ("RESIDUE_PATCH_MODE", "RESIDUE_ENABLE_DECODE_MEXT", "RESIDUE_FORCE_DECODE_MEXT", "RESIDUE_VLLM_MODEL_DIR"):
        monkeypatch.delenv(k, raising=False)
    env_contract.settings.cache_clear()
    from resinfer_b200.quant.vllm_integration import linear_method_v2 as L
    yield L.ResidueNvFp4LinearMethodV2
    env_contract.settings.cache_clear()


def _config(layers=None, k=256, ratio=0.25):
    meta = KM.build_kernel_metadata(layers or {}, residue_ratio=ratio, in_features={n: k for n in (layers or {})})
    return types.SimpleNamespace(group_size=16, is_checkpoint_nvfp4_serialized=True, _residue_metadata=meta)


def _layer(prefix):
    m = torch.nn.Module()
    m.prefix = prefix
    return m


def _load(layer, packed, indices=None):
    """What a checkpoint loader does: hand every tensor to the parameter's loader."""
    layer.weight.weight_loader(layer.weight, packed["weight"])
    layer.weight_scale.weight_loader(layer.weight_scale, packed["weight_scale_raw"])
    layer.weight_scale_2.weight_loader(layer.weight_scale_2, packed["weight_global_scale"].reshape(1))
    layer.input_scale.weight_loader(layer.input_scale, torch.tensor([0.5]))
    if indices is not None:
        layer.input_quantizer._salient_indices = indices.clone()


def _pack(n, k, sel):
    g = torch.Generator().manual_seed(n + k)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    p = weight_prep.quantize_weight_nvfp4(w, sel)
    p["weight_scale_raw"] = p["weight_scale_raw"].view(torch.float8_e4m3fn)     # as a checkpoint stores them
    return p


def test_extended_k_layer_column_parallel(method_cls, monkeypatch):
    monkeypatch.setenv("RESIDUE_ENABLE_DECODE_MEXT", "1")
    env_contract.settings.cache_clear()
    k, n = 256, 192
    name = "model.layers.0.self_attn.qkv_proj"
    sel = weight_prep.salient_indices_per8(k, 2)
    cfg = _config({name: sel}, k)
    method = method_cls(cfg, layer_prefix=name)
    layer = _layer(name)
    method.create_weights(layer, k, [n], k, n, torch.bfloat16)
    kx = k + sel.numel()
    assert layer.weight.shape == (n, kx // 2) and layer.weight.dtype == torch.uint8
    assert layer.weight_scale.shape == (n, kx // 16) and layer.weight_scale.dtype == torch.float8_e4m3fn
    assert layer.input_scale.shape == (1,) and layer.weight_scale_2.shape == (1,)
    assert not hasattr(layer, "_residue_shard_plan")
    packed = _pack(n, k, sel)
    _load(layer, packed, sel)
    method.process_weights_after_loading(layer)
    assert layer._runtime_mode == "extended_k" and layer._is_residue_layer
    assert layer.num_salient == sel.numel() and layer.original_in_features == k and layer.extended_in_features == kx
    from resinfer_b200.nvfp4.quant import indices_to_channel_masks
    assert torch.equal(layer.channel_mask, indices_to_channel_masks(sel, k))
    assert torch.equal(layer.weight_scale.view(torch.uint8).reshape(-1),
                       weight_prep.swizzle_scales_any(packed["weight_scale_raw"].view(torch.uint8)))
    # base-K buffer = the raw scale's first K/16 groups, swizzled on their own
    assert layer._decode_mext_layout_enabled and layer._mext_decode_k_base == k
    assert torch.equal(layer.weight_scale_base.view(torch.uint8).reshape(-1),
                       weight_prep.swizzle_scales_any(packed["weight_scale_raw"].view(torch.uint8)[:, :k // 16].contiguous()))
    gs_w = float(packed["weight_global_scale"])
    assert layer.alpha.shape == (1,) and abs(float(layer.alpha) - 0.5 * gs_w) < 1e-9 * max(1.0, gs_w)
    assert abs(float(layer.input_global_scale_inv) - 2.0) < 1e-7
    assert not hasattr(layer, "input_scale") and not hasattr(layer, "weight_scale_2")


def test_row_parallel_layer_gets_its_own_ranges(method_cls, monkeypatch):
    k, n, tp = 512, 128, 2
    name = "model.layers.0.mlp.down_proj"
    sel = weight_prep.salient_indices_per8(k, 2)                    # 128 salient channels, 64 per half
    cfg = _config({name: sel}, k)
    packed = _pack(n, k, sel)
    from resinfer_b200.quant.vllm_integration import linear_method_v2 as L
    from resinfer_b200.quant.vllm_integration.residue_tp import ResidueShardPlan
    for rank in range(tp):
        monkeypatch.setattr(L, "current_tp_rank", lambda r=rank: r)
        method = method_cls(cfg, layer_prefix=name)
        layer = _layer(name)
        method.create_weights(layer, k // tp, [n], k, n, torch.bfloat16, tp_rank=rank)
        plan = layer._residue_shard_plan
        assert isinstance(plan, ResidueShardPlan) and plan.tp_rank == rank and plan.k_ext_shard == (k + sel.numel()) // tp
        assert layer.weight.shape == (n, plan.k_ext_shard // 2)
        _load(layer, packed, sel)
        # the loader put [base_r | salient_r] of the checkpoint's [base | salient] here
        want = plan.gather(packed["weight"], 2)
        assert torch.equal(layer.weight.data, want)
        assert torch.equal(layer.weight_scale.data.view(torch.uint8),
                           plan.gather(packed["weight_scale_raw"].view(torch.uint8), 16))
        method.process_weights_after_loading(layer)
        local = plan.local_salient_indices(sel)
        assert layer.num_salient == local.numel() == sel.numel() // tp
        assert layer.original_in_features == k // tp
        assert int(local.min()) >= 0 and int(local.max()) < k // tp


def test_mext_r1_and_standard_modes(method_cls, monkeypatch):
    k, n = 256, 128
    r1 = "model.layers.0.mlp.gate_up_proj"
    cfg = _config({r1: torch.arange(k)}, k, ratio=1.0)               # every channel salient -> mext_r1
    assert KM.get_layer_metadata(cfg._residue_metadata, r1)["runtime_mode"] == "mext_r1"
    method = method_cls(cfg, layer_prefix=r1)
    layer = _layer(r1)
    method.create_weights(layer, k, [n // 2, n // 2], k, n, torch.bfloat16)
    assert layer.weight.shape == (n, k // 2) and layer.input_scale.shape == (2,)      # weight stays at K; two logical parts
    packed = _pack(n, k, None)
    layer.weight.data.copy_(packed["weight"])
    layer.weight_scale.data.copy_(packed["weight_scale_raw"])
    layer.weight_scale_2.data.copy_(torch.tensor([0.25, 0.75]))
    layer.input_scale.data.copy_(torch.tensor([0.125, 0.5]))
    method.process_weights_after_loading(layer)
    assert layer._runtime_mode == "mext_r1" and layer._is_residue_layer and layer.num_salient == 0
    assert layer.channel_mask is None and layer._decode_mext_layout_enabled and layer._mext_decode_k_base == k
    assert layer.weight_scale_base is layer.weight_scale
    assert abs(float(layer.alpha) - 0.5 * 0.75) < 1e-7                # merged projections share the largest scales
    # a layer without a sidecar record and without the decode switch is a plain NVFP4 layer
    plain = "model.layers.0.self_attn.o_proj"
    m2 = method_cls(cfg, layer_prefix=plain)
    l2 = _layer(plain)
    m2.create_weights(l2, k, [n], k, n, torch.bfloat16)
    _load(l2, packed)
    m2.process_weights_after_loading(l2)
    assert l2._runtime_mode == "standard" and not l2._is_residue_layer and not l2._decode_mext_layout_enabled
    # RESIDUE_PATCH_MODE=mext_r1 promotes plain projections by name
    monkeypatch.setenv("RESIDUE_PATCH_MODE", "mext_r1")
    env_contract.settings.cache_clear()
    m3 = method_cls(cfg, layer_prefix=plain)
    assert m3._runtime_mode(plain) == "mext_r1" and m3._runtime_mode("model.embed_tokens") == "standard"


def test_apply_hands_the_op_the_layer_state(method_cls, monkeypatch):
    monkeypatch.setenv("RESIDUE_ENABLE_DECODE_MEXT", "1")
    env_contract.settings.cache_clear()
    k, n = 256, 128
    name = "model.layers.0.self_attn.o_proj"
    sel = weight_prep.salient_indices_per8(k, 1)
    cfg = _config({name: sel}, k, ratio=0.125)
    method = method_cls(cfg, layer_prefix=name)
    layer = _layer(name)
    method.create_weights(layer, k, [n], k, n, torch.bfloat16)
    _load(layer, _pack(n, k, sel), sel)
    method.process_weights_after_loading(layer)
    seen = {}

    def fake_op(*args):
        seen["args"] = args
        return torch.zeros(args[0].shape[0], n, dtype=torch.bfloat16)

    monkeypatch.setattr(torch.ops.residue, "nvfp4_linear", fake_op, raising=False)
    x = torch.randn(2, 3, k).to(torch.bfloat16)
    bias = torch.ones(n, dtype=torch.bfloat16)
    y = method.apply(layer, x, bias)
    assert y.shape == (2, 3, n) and bool((y == 1).all())
    a = seen["args"]
    assert a[0].shape == (6, k) and a[1] is layer.weight and a[3] is layer.weight_scale and a[4] is layer.weight_scale_base
    assert a[5] is layer.channel_mask and a[6] is layer.alpha
    assert a[7:] == (k, sel.numel(), 0, n, True, False, False)          # k_base, S, padding, N, fold-eligible, swap, mext_r1
    assert method.apply(layer, x[:0], None).shape == (0, 3, n)         # empty input never reaches the op
    assert seen["args"] is a


def test_patch_installs_the_method_in_the_modelopt_loader(monkeypatch):
    pytest.importorskip("vllm")
    for k in ("RESIDUE_PATCH_MODE", "RESIDUE_ENABLE_DECODE_MEXT", "RESIDUE_VLLM_MODEL_DIR"):
        monkeypatch.delenv(k, raising=False)
    env_contract.settings.cache_clear()
    try:
        from vllm.model_executor.layers import linear
        from vllm.model_executor.layers.quantization.modelopt import ModelOptNvFp4Config
    except Exception as e:                                             # a vLLM that cannot be imported on this machine
        pytest.skip(f"vLLM's ModelOpt module is not importable here: {e}")
    from resinfer_b200.quant.vllm_integration import patch
    from resinfer_b200.quant.vllm_integration.linear_method_v2 import ResidueNvFp4LinearMethodV2
    saved = (ModelOptNvFp4Config.LinearMethodCls, ModelOptNvFp4Config.__init__, ModelOptNvFp4Config.get_quant_method,
             list(linear.WEIGHT_LOADER_V2_SUPPORTED), patch._installed_mode)
    try:
        patch._installed_mode = None
        assert patch.patch_vllm_modelopt() is True
        assert patch.is_patched() and ModelOptNvFp4Config.LinearMethodCls is ResidueNvFp4LinearMethodV2
        assert "ResidueNvFp4LinearMethodV2" in linear.WEIGHT_LOADER_V2_SUPPORTED
        assert patch.patch_vllm_modelopt() is False                   # second call: already installed
        with pytest.raises(ValueError, match="cannot change"):
            patch.patch_vllm_modelopt(version="mext_r1")
        with pytest.raises(ValueError, match="Unknown residue patch mode"):
            patch.patch_vllm_modelopt(version="v9")
    finally:
        (ModelOptNvFp4Config.LinearMethodCls, ModelOptNvFp4Config.__init__,
         ModelOptNvFp4Config.get_quant_method) = saved[:3]
        linear.WEIGHT_LOADER_V2_SUPPORTED[:] = saved[3]
        patch._installed_mode = saved[4]
        env_contract.settings.cache_clear()
