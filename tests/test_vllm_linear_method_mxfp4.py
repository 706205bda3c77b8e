"""The vLLM MXFP4 linear method on CPU: shape and tensor-parallel rules of ``create_weights``, the loaders'
interleave for row-parallel selective layers, the fused-group rules of method selection and the parser of the
checkpoint's quantisation block (reference: quant/vllm_integration/linear_method_mxfp4.py:22-276)."""
import types

import pytest
import torch

from resinfer_b200.quant import kernel_metadata as KM
from resinfer_b200.quant import weight_prep


@pytest.fixture(scope="module")
def M():
    from resinfer_b200.quant.vllm_integration import linear_method_mxfp4 as mod
    return mod


def _layer():
    return torch.nn.Module()


def test_create_weights_shapes_and_rules(M, monkeypatch):
    monkeypatch.delenv("RESIDUE_MXFP4_TP_EXPERIMENTAL", raising=False)
    k, n = 512, 256
    sel = weight_prep.salient_indices_per8(k, 2)
    rec = {"runtime_mode": "extended_k", "num_salient": sel.numel(), "salient_indices": sel.tolist()}
    m = M.ResidueMxfp4LinearMethod(rec, extended_dim=KM.padded_k(k, sel.numel()))
    layer = _layer()
    m.create_weights(layer, k, [n], k, n, torch.bfloat16)
    kp = KM.padded_k(k, sel.numel())
    assert m.mode == "selective" and layer.weight.shape == (n, kp // 2) and layer.weight_scale.shape == (n, kp // 32)
    assert layer.weight.dtype == torch.uint8 and layer.weight.input_dim == 1 and layer.weight.output_dim == 0
    with pytest.raises(ValueError, match="must be uint8"):
        layer.weight.weight_loader(layer.weight, torch.zeros(n, kp // 2))
    with pytest.raises(ValueError, match="K%128==0 and N%32==0"):
        M.ResidueMxfp4LinearMethod({}).create_weights(_layer(), 192, [n], 192, n, torch.bfloat16)
    with pytest.raises(ValueError, match="fp16 or bf16"):
        M.ResidueMxfp4LinearMethod({}).create_weights(_layer(), k, [n], k, n, torch.float32)
    with pytest.raises(ValueError, match="extended dimension does not match"):
        M.ResidueMxfp4LinearMethod(rec, extended_dim=kp + 128).create_weights(_layer(), k, [n], k, n, torch.bfloat16)
    with pytest.raises(ValueError, match="experimental"):
        M.ResidueMxfp4LinearMethod({}).create_weights(_layer(), k // 2, [n], k, n, torch.bfloat16)
    r1 = {"runtime_mode": "mext_r1", "num_salient": k, "salient_indices": list(range(k))}
    m1 = M.ResidueMxfp4LinearMethod(r1)
    l1 = _layer()
    m1.create_weights(l1, k, [n // 2, n // 2], k, n, torch.float16)
    assert m1.mode == "mext_r1" and m1.indices == () and l1.weight.shape == (n, k // 2) and l1._mxfp4_shards == 2
    with pytest.raises(RuntimeError, match="process_weights_after_loading"):
        m1.apply(l1, torch.zeros(1, k))


def test_row_parallel_selective_loader(M, monkeypatch):
    monkeypatch.setenv("RESIDUE_MXFP4_TP_EXPERIMENTAL", "1")
    k, n, tp = 1024, 64, 2
    sel = weight_prep.salient_indices_per8(k, 2)                    # 256 salient channels
    rec = {"runtime_mode": "extended_k", "num_salient": sel.numel(), "salient_indices": sel.tolist()}
    kx = k + sel.numel()
    full_w = torch.arange(n * (kx // 2), dtype=torch.int64).remainder(251).to(torch.uint8).reshape(n, kx // 2)
    full_s = torch.arange(n * (kx // 32), dtype=torch.int64).remainder(200).to(torch.uint8).reshape(n, kx // 32)
    for rank in range(tp):
        monkeypatch.setattr(M, "current_tp_rank", lambda r=rank: r)
        m = M.ResidueMxfp4LinearMethod(rec)
        layer = _layer()
        m.create_weights(layer, k // tp, [n], k, n, torch.bfloat16, tp_rank=rank)
        plan = layer._mxfp4_shard_plan
        assert plan.tp_rank == rank and plan.k_alignment == 128
        kp = KM.padded_k(k // tp, plan.salient_shard)
        assert layer.weight.shape == (n, kp // 2)
        layer.weight.weight_loader(layer.weight, full_w)
        layer.weight_scale.weight_loader(layer.weight_scale, full_s)
        assert torch.equal(layer.weight.data, plan.gather(full_w, 2))
        assert torch.equal(layer.weight_scale.data, plan.gather(full_s, 32))
        assert layer._mxfp4_loaded == {"weight": {None}, "weight_scale": {None}}
    with pytest.raises(ValueError, match="both input and output"):
        M.ResidueMxfp4LinearMethod({}).create_weights(_layer(), k // 2, [n // 2], k, n, torch.bfloat16)


def test_method_selection_rules_of_fused_layers(M):
    k = 256
    sel = weight_prep.salient_indices_per8(k, 2)
    base = "model.layers.0.self_attn."
    layers = {base + p: sel for p in ("q_proj", "k_proj", "v_proj")}
    meta = KM.build_kernel_metadata(layers, residue_ratio=0.25, in_features={n: k for n in layers})
    cfg = types.SimpleNamespace(_residue_metadata=meta)
    none = lambda name: False                                        # noqa: E731
    m = M.select_method(cfg, base + "qkv_proj", none)
    assert isinstance(m, M.ResidueMxfp4LinearMethod) and m.metadata["num_salient"] == sel.numel()
    assert M.select_method(cfg, base + "qkv_proj", lambda name: name.endswith(("q_proj", "k_proj", "v_proj"))) is None
    with pytest.raises(ValueError, match="partially quantized fused group"):
        M.select_method(cfg, base + "qkv_proj", lambda name: name.endswith("q_proj"))
    broken = {"layers": {base + "q_proj": meta["layers"][base + "q_proj"]}, "extended_linear_dims": {}}
    with pytest.raises(ValueError, match="partially specified residue fused group"):
        M.select_method(types.SimpleNamespace(_residue_metadata=broken), base + "qkv_proj", none)
    other = dict(meta["layers"][base + "q_proj"], num_salient=1)
    mixed = {"layers": dict(meta["layers"], **{base + "k_proj": other}), "extended_linear_dims": {}}
    with pytest.raises(ValueError, match="must share residue metadata"):
        M.select_method(types.SimpleNamespace(_residue_metadata=mixed), base + "qkv_proj", none)
    plain = M.select_method(types.SimpleNamespace(_residue_metadata={}), "model.layers.0.mlp.down_proj", none)
    assert plain.metadata == {} and plain.extended_dim is None


def test_quantisation_block_parser(M):
    ok = {"quantization": {"quant_algo": "MXFP4", "group_size": 32, "exclude_modules": ["lm_head"]}}
    assert M.parse_modelopt_mxfp4_config(ok) == ["lm_head"]
    for bad, text in (({"quant_algo": "NVFP4"}, "requires quant_algo=MXFP4"), ({"quant_algo": "MXFP4", "group_size": 16}, "group_size=32"),
                      ({"quant_algo": "MXFP4", "kv_cache_quant_algo": "FP8"}, "quantized KV cache"),
                      ({"quant_algo": "MXFP4", "exclude_modules": "lm_head"}, "list of strings")):
        with pytest.raises(ValueError, match=text):
            M.parse_modelopt_mxfp4_config(bad)
    if M.ModelOptMxfp4Config is not None:
        cfg = M.ModelOptMxfp4Config.from_config(ok)
        assert cfg.get_name() == "modelopt_mxfp4" and cfg.get_min_capability() == 100


def test_residue_spec():
    k = 256
    assert KM.residue_spec({}, k, 64) == {"mode": "standard", "input_size": k, "output_size": 64}
    r1 = KM.residue_spec({"runtime_mode": "mext_r1", "salient_indices": list(range(k))}, k, 64)
    assert r1["mode"] == "mext_r1" and "indices" not in r1
    sel = weight_prep.salient_indices_per8(k, 1).tolist()
    assert KM.residue_spec({"salient_indices": sel}, k, 64)["mode"] == "selective"
    with pytest.raises(ValueError, match="num_salient disagrees"):
        KM.residue_spec({"salient_indices": sel, "num_salient": 3}, k, 64)
    with pytest.raises(ValueError, match="every input channel"):
        KM.residue_spec({"runtime_mode": "mext_r1", "salient_indices": sel}, k, 64)
    with pytest.raises(ValueError, match="invalid residue runtime mode"):
        KM.residue_spec({"runtime_mode": "standard", "salient_indices": sel}, k, 64)
