"""Sidecar metadata (``residue_kernel_metadata.json``) as the vLLM linear methods see it: looked up through
the quantisation config object, read once per config.

Mirrors the reference's quant/vllm_integration/metadata.py:23-100 (``get_residue_metadata``,
``get_layer_metadata``, ``get_extended_dim`` taking the quant config); the name resolution itself (aliases,
fused projections, short-name suffix matching) lives in ``resinfer_b200.quant.kernel_metadata``.
"""
from __future__ import annotations

import os
from pathlib import Path

from .. import kernel_metadata as KM


def get_residue_metadata(quant_config, *, require_local: bool = False) -> dict:
    """The sidecar of the model the config belongs to.  The directory is ``$RESIDUE_VLLM_MODEL_DIR`` or, when
    vLLM is running, the model path of its current config.  A plain checkpoint without a local directory
    yields ``{}`` unless ``require_local`` (or the environment variable) demands one."""
    data = getattr(quant_config, "_residue_metadata", None)
    if data is not None:
        return data
    model_dir = os.environ.get("RESIDUE_VLLM_MODEL_DIR")
    if not model_dir:
        try:
            from vllm.config import get_current_vllm_config_or_none
            cfg = get_current_vllm_config_or_none()
            model_dir = cfg.model_config.model if cfg and cfg.model_config else None
        except Exception:                                   # vLLM absent, or no config in flight
            model_dir = None
    if not model_dir or not Path(model_dir).is_dir():
        if not require_local and not os.environ.get("RESIDUE_VLLM_MODEL_DIR"):
            return {}                                       # not cached: the path may resolve later
        raise ValueError("Residue metadata requires a local model directory; "
                         "set RESIDUE_VLLM_MODEL_DIR to the checkpoint directory")
    data = KM.load_residue_metadata(model_dir)
    quant_config._residue_metadata = data
    return data


def get_layer_metadata(quant_config, layer_name: str) -> dict | None:
    return KM.get_layer_metadata(get_residue_metadata(quant_config), layer_name)


def get_extended_dim(quant_config, layer_name: str) -> int | None:
    return KM.get_extended_dim(get_residue_metadata(quant_config), layer_name)
