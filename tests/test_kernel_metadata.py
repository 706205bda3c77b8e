"""The on-disk contract of the linear path (CPU): sidecar round trip, layer-name resolution, MXFP4 layer
specifications and the offline packer's tensors against the op contract."""
import json

import numpy as np
import pytest
import torch

import oracle as O
from resinfer_b200.quant import kernel_metadata as KM
from resinfer_b200.quant import weight_prep


def test_sidecar_round_trip_and_lookup(tmp_path):
    k = 256
    sel = weight_prep.salient_indices_per8(k, 2)
    layers = {"model.layers.0.self_attn.q_proj": sel, "model.layers.0.self_attn.k_proj": sel,
              "model.layers.0.self_attn.v_proj": sel, "model.layers.0.mlp.down_proj": torch.arange(512)}
    meta = KM.build_kernel_metadata(layers, residue_ratio=0.25, in_features={n: (512 if "down" in n else k) for n in layers})
    assert meta["layers"]["model.layers.0.mlp.down_proj"]["runtime_mode"] == "mext_r1"      # every channel salient
    assert meta["layers"]["model.layers.0.self_attn.q_proj"]["runtime_mode"] == "extended_k"
    assert meta["extended_linear_dims"]["model.layers.0.self_attn.q_proj"] == k + sel.numel()
    assert "model.layers.0.mlp.down_proj" not in meta["extended_linear_dims"]              # MEXT keeps K
    paths = KM.write_kernel_metadata(meta, tmp_path, mask_dims={n: k for n in layers if "down" not in n})
    assert paths["metadata_json"].name == "residue_kernel_metadata.json"
    back = KM.load_residue_metadata(tmp_path)
    assert back == json.loads(json.dumps(meta))
    masks = torch.load(paths["channel_masks"])
    assert masks["model.layers.0.self_attn.q_proj"].sum().item() == sel.numel()
    # fused runtime name resolves to its checkpoint constituents; Qwen3.5 prefix aliasing works both ways
    rec = KM.get_layer_metadata(back, "model.layers.0.self_attn.qkv_proj")
    assert rec["num_salient"] == sel.numel()
    assert KM.get_extended_dim(back, "model.layers.0.self_attn.qkv_proj") == k + sel.numel()
    assert "language_model.model.layers.0.mlp.gate_proj" in KM.get_residue_layer_candidates(
        "model.language_model.layers.0.mlp.gate_up_proj")
    assert KM.load_residue_metadata(tmp_path / "missing") == {}
    (tmp_path / "bad.json").write_text("[1, 2]")
    with pytest.raises(ValueError, match="must be an object"):
        KM.read_residue_metadata_json(tmp_path / "bad.json")
    with pytest.raises(ValueError, match="strictly increasing"):
        KM.build_kernel_metadata({"x": [3, 1]})
    with pytest.raises(ValueError, match="outside K"):
        KM.build_kernel_metadata({"x": [1, 999]}, in_features={"x": 256})


def test_mxfp4_layer_specs():
    k = 256
    idx = weight_prep.salient_indices_per8(k, 2).tolist()
    KM.validate_layer({"mode": "selective", "input_size": k, "output_size": 64, "indices": idx})
    KM.validate_layer({"mode": "mext_r1", "input_size": k, "output_size": 64})
    for bad in ({"mode": "selective", "input_size": k, "output_size": 64, "indices": idx[:-1]},
                {"mode": "selective", "input_size": k, "output_size": 64, "indices": sorted(idx, reverse=True)},
                {"mode": "standard", "input_size": k, "output_size": 64, "indices": idx},
                {"mode": "standard", "input_size": 100, "output_size": 64},
                {"mode": "other", "input_size": k, "output_size": 64}):
        with pytest.raises(ValueError):
            KM.validate_layer(bad)
    assert KM.padded_k(5120, 640) == 5760 and KM.padded_k(5120, 100) == 5248
    spec = {"mode": "mext_r1", "input_size": k}
    fused = KM.fuse_projection_specs({"m.q_proj": dict(spec, output_size=64), "m.k_proj": dict(spec, output_size=32),
                                      "m.v_proj": dict(spec, output_size=32), "m.o_proj": dict(spec, output_size=64)})
    assert fused == {"m.qkv_proj": dict(spec, output_size=128), "m.o_proj": dict(spec, output_size=64)}
    with pytest.raises(ValueError, match="partially quantized"):
        KM.fuse_projection_specs({"m.q_proj": dict(spec, output_size=64)})
    with pytest.raises(ValueError, match="must share"):
        KM.fuse_projection_specs({"m.gate_proj": dict(spec, output_size=64),
                                  "m.up_proj": dict(spec, output_size=64, input_size=512)})


def test_packer_matches_the_op_contract(tmp_path):
    """Packed tensors carry [W | W[:, salient]] for extended_k layers, the base K for mext_r1 layers, and
    dequantise back to the dense weight within FP4 error; a sidecar that lies about the width is caught."""
    n, k = 64, 256
    w = torch.from_numpy(O.make_weight(n, k, seed=3))
    sel = weight_prep.salient_indices_per8(k, 2)
    dense = {"l.q_proj.weight": w, "l.o_proj.weight": w.clone(), "l.norm.weight": torch.ones(k)}
    meta = KM.build_kernel_metadata({"l.q_proj": sel, "l.o_proj": torch.arange(k)}, in_features={"l.q_proj": k, "l.o_proj": k})
    packed = KM.pack_checkpoint(dense, meta, tmp_path, fmt="nvfp4")
    assert set(packed) == {"l.q_proj", "l.o_proj"}
    q, o = packed["l.q_proj"], packed["l.o_proj"]
    assert q["weight"].shape == (n, (k + sel.numel()) // 2) and q["num_salient"] == sel.numel() and q["k_base"] == k
    assert o["weight"].shape == (n, k // 2) and o["num_salient"] == 0                      # MEXT: not widened
    wd = O.dequant_operand(q["weight"].numpy(), q["weight_scale"].numpy(), "nvfp4") * float(q["weight_global_scale"])
    ext = np.concatenate([w.numpy(), w.numpy()[:, sel.numpy()]], axis=1)
    assert np.linalg.norm(wd - ext) / np.linalg.norm(ext) < 0.12
    saved = torch.load(tmp_path / KM.PACKED_FILE)
    assert torch.equal(saved["l.q_proj"]["weight"], q["weight"])
    assert KM.load_residue_metadata(tmp_path)["layers"]["l.o_proj"]["runtime_mode"] == "mext_r1"
    assert KM.validate_packed_widths(packed, meta) == 1
    lying = json.loads(json.dumps(meta))
    lying["layers"]["l.q_proj"]["num_salient"] = 2 * sel.numel()
    with pytest.raises(AssertionError, match="not widened"):
        KM.validate_packed_widths(packed, lying)
    mx = KM.pack_linear(w, meta["layers"]["l.q_proj"], fmt="mxfp4")
    assert mx["weight"].shape == (n, KM.padded_k(k, sel.numel()) // 2)
    with pytest.raises(ValueError, match="multiple of 64"):
        KM.pack_linear(w, {"runtime_mode": "extended_k", "salient_indices": [0, 8, 16]}, fmt="nvfp4")
