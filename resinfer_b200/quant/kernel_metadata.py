"""On-disk contract either side of the linear hot path: the ``residue_kernel_metadata.json`` sidecar
and an offline packer that turns dense weights into the tensors ``residue::nvfp4_linear`` /
``residue::mxfp4_linear`` consume.

Format of the sidecar (what the reference writes in quant/modelopt_integration/kernel_metadata.py:86-135,
199-220 and reads in quant/vllm_integration/metadata.py:13-100)::

    {"layers": {"<hf layer name>": {"salient_indices": [...], "num_salient": S,
                                     "runtime_mode": "extended_k" | "mext_r1"}},
     "global": {"residue_ratio": r, "block_size": 8},
     "extended_linear_dims": {"<layer name>": K + S}}

``runtime_mode == "mext_r1"`` layers keep their weight at the original K (MEXT fold), ``extended_k`` layers
carry ``[W | W[:, salient]]``.  Layer lookups accept the runtime's fused names (``qkv_proj``,
``gate_up_proj`` ...) and the Qwen3.5 prefix aliasing, like the reference's reader.  The MXFP4 layer
specification and its checks follow quant/kernel_metadata.py:7-47.

Nothing here touches the GPU: the packer runs wherever the weights live (``weight_prep`` is plain torch).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from . import weight_prep

SIDE_CAR = "residue_kernel_metadata.json"
PACKED_FILE = "residue_packed_linears.pt"

# runtime (fused) projection -> checkpoint constituents
FUSED_PROJECTIONS = {
    "qkv_proj": ("q_proj", "k_proj", "v_proj"),
    "gate_up_proj": ("gate_proj", "up_proj"),
    "in_proj_qkvz": ("in_proj_qkv", "in_proj_z"),
    "in_proj_ba": ("in_proj_b", "in_proj_a"),
}
_PREFIX_ALIASES = (("language_model.model.", "model.language_model."),
                   ("model.language_model.", "language_model.model."))


# ------------------------------------------------------------------------------------------------
# sidecar: build, write, read
# ------------------------------------------------------------------------------------------------
def is_mext_r1_layer(num_salient: int, in_features: int) -> bool:
    """A layer whose every input channel is salient runs as MEXT (ratio 1.0) and is never K-extended."""
    return in_features > 0 and num_salient == in_features


def build_kernel_metadata(layers: dict, *, residue_ratio: float = 0.25, block_size: int = 8,
                          in_features: dict | None = None) -> dict:
    """``layers`` maps a layer name to its salient channel indices (tensor / sequence) or to a ready
    record.  ``in_features`` (name -> K) lets ratio-1.0 layers be recognised and fills
    ``extended_linear_dims`` for the K-extended ones."""
    meta = {"layers": {}, "global": {"residue_ratio": float(residue_ratio), "block_size": int(block_size)},
            "extended_linear_dims": {}}
    for name, value in layers.items():
        if isinstance(value, dict):
            rec = dict(value)
            idx = [int(i) for i in rec.get("salient_indices", [])]
        else:
            idx = [int(i) for i in (value.tolist() if hasattr(value, "tolist") else value)]
            rec = {}
        if any(a >= b for a, b in zip(idx, idx[1:])):
            raise ValueError(f"{name}: salient indices must be strictly increasing")
        rec["salient_indices"] = idx
        rec["num_salient"] = len(idx)
        k = None if in_features is None else in_features.get(name)
        if "runtime_mode" not in rec:
            rec["runtime_mode"] = "mext_r1" if k is not None and is_mext_r1_layer(len(idx), int(k)) else "extended_k"
        if rec["runtime_mode"] not in ("extended_k", "mext_r1"):
            raise ValueError(f"{name}: unknown runtime_mode {rec['runtime_mode']!r}")
        if k is not None:
            if idx and idx[-1] >= int(k):
                raise ValueError(f"{name}: salient index {idx[-1]} outside K={k}")
            if rec["runtime_mode"] == "extended_k" and idx:
                meta["extended_linear_dims"][name] = int(k) + len(idx)
        meta["layers"][name] = rec
    return meta


def write_kernel_metadata(metadata: dict, export_dir, *, mask_dims: dict | None = None) -> dict:
    """Write the sidecar (and, when ``mask_dims`` gives K per layer, ``channel_masks.pt`` with one bool
    mask per layer).  Returns the paths written."""
    export_dir = Path(export_dir)
    export_dir.mkdir(parents=True, exist_ok=True)
    path = export_dir / SIDE_CAR
    path.write_text(json.dumps(metadata, indent=2, ensure_ascii=False), encoding="utf-8")
    written = {"metadata_json": path}
    masks = {}
    for name, k in (mask_dims or {}).items():
        rec = metadata.get("layers", {}).get(name)
        if rec is None or k is None or not rec.get("salient_indices"):
            continue
        idx = torch.tensor(rec["salient_indices"], dtype=torch.long)
        if int(idx.max()) >= int(k):
            continue
        mask = torch.zeros(int(k), dtype=torch.bool)
        mask[idx] = True
        masks[name] = mask
    if masks:
        written["channel_masks"] = export_dir / "channel_masks.pt"
        torch.save(masks, written["channel_masks"])
    return written


def read_residue_metadata_json(metadata_path) -> dict:
    """Read one sidecar; file and JSON errors propagate, a non-object is rejected."""
    with open(metadata_path, encoding="utf-8") as f:
        data = json.load(f)
    if not isinstance(data, dict):
        raise ValueError(f"Residue metadata must be an object: {metadata_path}")
    return data


def load_residue_metadata(model_dir) -> dict:
    """The sidecar of a checkpoint directory, or {} when the checkpoint has none (plain NVFP4)."""
    try:
        return read_residue_metadata_json(Path(model_dir) / SIDE_CAR)
    except FileNotFoundError:
        return {}


# ------------------------------------------------------------------------------------------------
# name resolution
# ------------------------------------------------------------------------------------------------
def _layer_aliases(layer_name: str) -> list[str]:
    names = [layer_name]
    for source, target in _PREFIX_ALIASES:
        if layer_name.startswith(source):
            names.append(target + layer_name[len(source):])
            break
    return names


def get_fused_hf_candidates(layer_name: str) -> list[list[str]]:
    """Checkpoint constituents of a fused runtime projection, one group per prefix spelling."""
    groups = []
    for cand in _layer_aliases(layer_name):
        parent, dot, leaf = cand.rpartition(".")
        if leaf in FUSED_PROJECTIONS:
            groups.append([parent + dot + part for part in FUSED_PROJECTIONS[leaf]])
    return groups


def get_residue_layer_candidates(layer_name: str) -> list[str]:
    """Names to try for a runtime layer: itself and its aliases first, then the fused constituents."""
    names = _layer_aliases(layer_name)
    for group in get_fused_hf_candidates(layer_name):
        names.extend(group)
    return list(dict.fromkeys(names))


def get_layer_metadata(metadata: dict, layer_name: str) -> dict | None:
    layers = metadata.get("layers", {})
    for cand in get_residue_layer_candidates(layer_name):
        rec = layers.get(cand)
        if rec:
            return rec
    return None


def get_extended_dim(metadata: dict, layer_name: str) -> int | None:
    """Checkpoint input width K + S of a K-extended layer (suffix matching kept for old short names)."""
    dims = metadata.get("extended_linear_dims", {})
    for cand in get_residue_layer_candidates(layer_name):
        if cand in dims:
            return dims[cand]
    for key, dim in dims.items():
        if key.endswith(layer_name) or layer_name.endswith(key):
            return dim
    return None


# ------------------------------------------------------------------------------------------------
# MXFP4 layer specification
# ------------------------------------------------------------------------------------------------
def padded_k(k: int, selected: int = 0) -> int:
    return (k + selected + 127) // 128 * 128


def validate_layer(spec: dict) -> None:
    """MXFP4 execution contract of one layer: {"mode", "input_size", "output_size"[, "indices"]}."""
    k, n = spec.get("input_size"), spec.get("output_size")
    if type(k) is not int or k <= 0 or k % 128 or type(n) is not int or n <= 0 or n % 32:
        raise ValueError("MXFP4 requires positive input_size%128==0 and output_size%32==0")
    mode = spec.get("mode")
    if mode not in ("standard", "selective", "mext_r1"):
        raise ValueError(f"unsupported MXFP4 mode {mode}")
    idx = spec.get("indices", [])
    if mode != "selective":
        if idx:
            raise ValueError("indices are only stored for selective mode")
        return
    per8 = {k // 8: 1, k // 4: 2, k // 2: 4}.get(len(idx))
    ok = per8 is not None and all(type(i) is int and 0 <= i < k for i in idx)
    ok = ok and all(a < b for a, b in zip(idx, idx[1:]))
    ok = ok and all(v // 8 == j // per8 for j, v in enumerate(idx))
    if not ok:
        raise ValueError("selective indices must be sorted, unique, in range, with exactly 1/2/4 selections "
                         "per group of 8")


def residue_spec(metadata: dict | None, input_size: int, output_size: int) -> dict:
    """A sidecar layer record -> the MXFP4 execution contract of ``validate_layer`` (reference:
    quant/kernel_metadata.py:79-100).  ``mext_r1`` records must list every input channel in order and carry
    no indices in the spec; ``extended_k`` records become ``selective``; records without indices are ``standard``."""
    metadata = metadata or {}
    indices = list(metadata.get("salient_indices", []))
    if metadata.get("num_salient", len(indices)) != len(indices):
        raise ValueError("num_salient disagrees with salient_indices")
    runtime_mode = metadata.get("runtime_mode", "extended_k" if indices else "standard")
    if runtime_mode == "mext_r1":
        if indices != list(range(input_size)):
            raise ValueError("mext_r1 requires every input channel in order")
        mode, indices = "mext_r1", []
    elif runtime_mode == "extended_k" and indices:
        mode = "selective"
    elif runtime_mode == "standard" and not indices:
        mode = "standard"
    else:
        raise ValueError(f"invalid residue runtime mode: {runtime_mode}")
    spec = {"mode": mode, "input_size": input_size, "output_size": output_size}
    if indices:
        spec["indices"] = indices
    validate_layer(spec)
    return spec


def fuse_projection_specs(layers: dict) -> dict:
    """Merge the checkpoint constituents of fused projections; they must agree on everything but N."""
    out = dict(layers)
    for target, parts in FUSED_PROJECTIONS.items():
        parents = sorted({name.rsplit(".", 1)[0] for name in layers if name.rsplit(".", 1)[-1] in parts})
        for parent in parents:
            names = [f"{parent}.{p}" for p in parts]
            if any(nm not in layers for nm in names):
                raise ValueError(f"partially quantized fused group is unsupported: {names}")
            shared = [{k: v for k, v in layers[nm].items() if k != "output_size"} for nm in names]
            if any(s != shared[0] for s in shared[1:]):
                raise ValueError(f"fused group must share mode, indices, input size: {names}")
            for nm in names:
                del out[nm]
            out[f"{parent}.{target}"] = dict(shared[0], output_size=sum(layers[nm]["output_size"] for nm in names))
    return out


# ------------------------------------------------------------------------------------------------
# offline packer
# ------------------------------------------------------------------------------------------------
def pack_linear(weight: torch.Tensor, record: dict | None, fmt: str = "nvfp4") -> dict:
    """Dense ``[N, K]`` weight + its sidecar record -> the tensors of the linear ops.  ``extended_k``
    layers are widened to ``[W | W[:, salient]]`` before quantisation, ``mext_r1`` and plain layers keep K."""
    idx = None
    if record and record.get("runtime_mode", "extended_k") == "extended_k" and record.get("salient_indices"):
        idx = torch.tensor(record["salient_indices"], dtype=torch.long, device=weight.device)
    if fmt == "nvfp4":
        if weight.shape[1] % 64 or (idx is not None and idx.numel() % 64):
            raise ValueError("NVFP4 needs K % 64 == 0 and a K extension that is a multiple of 64")
        return weight_prep.quantize_weight_nvfp4(weight, idx)
    if fmt == "mxfp4":
        if weight.shape[1] % 128 or weight.shape[0] % 32:
            raise ValueError("MXFP4 requires input_size%128==0 and output_size%32==0")
        return weight_prep.quantize_weight_mxfp4(weight, idx)
    raise ValueError(f"unknown format {fmt!r}")


def pack_checkpoint(dense: dict, metadata: dict, export_dir, fmt: str = "nvfp4") -> dict:
    """Pack every 2-D ``<layer>.weight`` of ``dense`` (a state dict), write ``residue_packed_linears.pt``
    next to the sidecar and return {layer: packed tensors}.  Layers without a record are packed plain."""
    export_dir = Path(export_dir)
    export_dir.mkdir(parents=True, exist_ok=True)
    packed = {}
    for key, w in dense.items():
        if not key.endswith(".weight") or w.dim() != 2:
            continue
        name = key[: -len(".weight")]
        packed[name] = pack_linear(w, get_layer_metadata(metadata, name), fmt)
    validate_packed_widths(packed, metadata, fmt)
    torch.save({n: {k: (v.cpu() if hasattr(v, "cpu") else v) for k, v in p.items()} for n, p in packed.items()},
               export_dir / PACKED_FILE)
    write_kernel_metadata(metadata, export_dir)
    return packed


def validate_packed_widths(packed: dict, metadata: dict, fmt: str = "nvfp4") -> int:
    """Every ``extended_k`` layer must really be widened: packed width (K + S) / 2 bytes (NVFP4) or the
    128-padded equivalent (MXFP4).  A sidecar that declares an extension the weights do not carry would
    make the kernels read past the weight rows.  Returns how many layers were checked (the check of the
    reference's export validation, export/validation.py:32-81, on packed tensors instead of safetensors)."""
    bad, checked = [], 0
    for name, rec in metadata.get("layers", {}).items():
        if not isinstance(rec, dict) or rec.get("runtime_mode") != "extended_k":
            continue
        s = int(rec.get("num_salient", 0))
        p = packed.get(name)
        if s <= 0 or p is None:
            continue
        k = int(p["k_base"])
        want = (k + s) // 2 if fmt == "nvfp4" else padded_k(k, s) // 2
        checked += 1
        if p["weight"].shape[1] != want or int(p["num_salient"]) != s:
            bad.append(f"{name}: num_salient={s} K={k} expected packed width {want}, got {p['weight'].shape[1]}")
    if bad:
        raise AssertionError(f"{len(bad)} of {checked} extended_k layers are not widened as the metadata says. "
                             f"First: {bad[0]}")
    return checked


__all__ = [
    "FUSED_PROJECTIONS", "SIDE_CAR", "PACKED_FILE", "build_kernel_metadata", "write_kernel_metadata",
    "read_residue_metadata_json", "load_residue_metadata", "get_fused_hf_candidates",
    "get_residue_layer_candidates", "get_layer_metadata", "get_extended_dim", "padded_k", "validate_layer",
    "fuse_projection_specs", "pack_linear", "pack_checkpoint", "validate_packed_widths", "is_mext_r1_layer",
]
