"""From disk through the ops: a synthetic checkpoint is packed with ``quant/kernel_metadata.py`` (packed FP4
weights + ``residue_kernel_metadata.json`` sidecar, the on-disk contract of the reference:
quant/modelopt_integration/kernel_metadata.py:86-135, quant/vllm_integration/metadata.py:13-100), read back
from the files alone, and every layer is run through ``residue::nvfp4_linear`` / ``residue::mxfp4_linear``
with the arguments a loader derives from the sidecar (base K, number of salient channels, channel mask,
runtime mode).  Each output is checked against the oracle's contraction of the same codes (BF16 rounding
tolerance) and against the dense BF16 product (quantisation error)."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _export(tmp_path, fmt):
    from resinfer_b200.quant import kernel_metadata as KM
    from resinfer_b200.quant import weight_prep
    k, n = 1024, 384
    dense = {"model.layers.0.self_attn.o_proj.weight": torch.from_numpy(O.make_weight(n, k, seed=21)),
             "model.layers.0.mlp.down_proj.weight": torch.from_numpy(O.make_weight(n, k, seed=22)),
             "model.layers.0.input_layernorm.weight": torch.ones(k)}
    sel = weight_prep.salient_indices_per8(k, 2)                       # ratio 0.25 -> K-extended layer
    layers = {"model.layers.0.self_attn.o_proj": sel,                  # extended_k
              "model.layers.0.mlp.down_proj": torch.arange(k)}         # every channel salient -> mext_r1
    meta = KM.build_kernel_metadata(layers, residue_ratio=0.25, in_features={name: k for name in layers})
    KM.pack_checkpoint(dense, meta, tmp_path, fmt=fmt)
    return dense, k, n


@pytest.mark.parametrize("m", [8, 200])
def test_nvfp4_checkpoint_from_disk_through_the_op(cuda_device, tmp_path, m):
    from resinfer_b200.nvfp4.quant import indices_to_channel_masks
    from resinfer_b200.quant import kernel_metadata as KM
    from resinfer_b200.quant.vllm_integration import residue_linear_op  # noqa: F401  (registers the op)
    dense, k, n = _export(tmp_path, "nvfp4")
    dev = cuda_device
    # ---- a loader that knows nothing but the export directory
    meta = KM.load_residue_metadata(tmp_path)
    packed = torch.load(tmp_path / KM.PACKED_FILE)
    assert KM.validate_packed_widths(packed, meta) == 1
    x_np = O.make_activation(m, k, seed=5)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    gs = float(np.abs(x_np).max()) / (6 * 448)
    gi = torch.tensor([1 / gs], dtype=torch.float32, device=dev)
    for name, p in packed.items():
        rec = KM.get_layer_metadata(meta, name)
        ratio1 = rec["runtime_mode"] == "mext_r1"
        s = 0 if ratio1 else int(rec["num_salient"])
        assert KM.get_extended_dim(meta, name) == (None if ratio1 else k + s)
        idx = torch.tensor(rec["salient_indices"], dtype=torch.long, device=dev)
        mask = torch.zeros(1, dtype=torch.uint8, device=dev) if ratio1 else indices_to_channel_masks(idx, k)
        w, wsf, wsf_base = p["weight"].to(dev), p["weight_scale"].to(dev), p["weight_scale_base"].to(dev)
        alpha = (p["weight_global_scale"].to(dev) * gs).float().reshape(1)
        y = torch.ops.residue.nvfp4_linear(x, w, gi, wsf, wsf_base, mask, alpha, int(p["k_base"]), s, 0, n, True, False,
                                           ratio1)
        assert y.shape == (m, n) and y.dtype == torch.bfloat16
        # the oracle's contraction of the codes the route produces: fold (row pair) up to 128 tokens (512 for a
        # ratio-1 layer), masked K extension above
        wd = O.dequant_operand(p["weight"].numpy(), p["weight_scale"].numpy(), "nvfp4")
        if ratio1 or m <= 128:
            codes, sf, _ = O.nvfp4_quant_mext(x_np, np.float32(1 / gs), 1)
            a = O.dequant_operand(codes, sf, "nvfp4")
            ref = O.fp4_linear_reference(a[0::2] + a[1::2], wd[:, :k], float(alpha.item()), False)
        else:
            codes, sf = O.nvfp4_quant_kext(x_np, np.float32(1 / gs), mask.cpu().numpy(), 2)[:2]
            ref = O.fp4_linear_reference(O.dequant_operand(codes, sf, "nvfp4"), wd, float(alpha.item()), False)
        got = y.float().cpu().numpy()
        assert rel_fro(got, ref) < 5e-3, name                  # BF16 output; quantiser reciprocals are approximate
        w_dense = dense[name + ".weight"].numpy().astype(np.float64)
        assert rel_fro(got, x_np.astype(np.float64) @ w_dense.T) < 0.15, name


def test_mxfp4_checkpoint_from_disk_through_the_op(cuda_device, tmp_path):
    from resinfer_b200.nvfp4.mxfp4 import prepare_indices
    from resinfer_b200.quant import kernel_metadata as KM
    from resinfer_b200.quant import mxfp4_linear  # noqa: F401  (registers the op)
    dense, k, n = _export(tmp_path, "mxfp4")
    dev = cuda_device
    meta = KM.load_residue_metadata(tmp_path)
    packed = torch.load(tmp_path / KM.PACKED_FILE)
    assert KM.validate_packed_widths(packed, meta, fmt="mxfp4") == 1
    m = 40
    x_np = O.make_activation(m, k, seed=6)
    x = torch.from_numpy(x_np).to(torch.bfloat16).to(dev)
    for name, p in packed.items():
        rec = KM.get_layer_metadata(meta, name)
        if rec["runtime_mode"] == "mext_r1":
            mode = "mext_r1"
            idx = torch.zeros(0, dtype=torch.int32, device=dev)
            masks = torch.zeros(0, dtype=torch.uint8, device=dev)
            KM.validate_layer({"mode": mode, "input_size": k, "output_size": n})
        else:
            mode = "selective"
            KM.validate_layer({"mode": mode, "input_size": k, "output_size": n, "indices": rec["salient_indices"]})
            idx, masks = prepare_indices(torch.tensor(rec["salient_indices"]), k, dev)
            assert p["weight"].shape[1] == KM.padded_k(k, int(rec["num_salient"])) // 2
        y = torch.ops.residue.mxfp4_linear(x, p["weight"].to(dev), p["weight_scale"].to(dev), idx, masks, mode,
                                           torch.bfloat16, None)
        got = y.float().cpu().numpy()
        wd = O.dequant_operand(p["weight"].numpy(), p["weight_scale"].numpy(), "mxfp4")
        if mode == "mext_r1":
            codes, sf = O.mxfp4_quant_mext(x_np)[:2]
            a = O.dequant_operand(codes, sf, "mxfp4")
            ref = O.fp4_linear_reference(a[0::2] + a[1::2], wd, 1.0, False)
        else:
            codes, sf = O.mxfp4_quant_selective(x_np, masks.cpu().numpy(), 2, kp=wd.shape[1])[:2]
            ref = O.fp4_linear_reference(O.dequant_operand(codes, sf, "mxfp4"), wd, 1.0, False)
        assert rel_fro(got, ref) < 5e-3, name
        w_dense = dense[name + ".weight"].numpy().astype(np.float64)
        assert rel_fro(got, x_np.astype(np.float64) @ w_dense.T) < 0.2, name
