"""Kernel loading and the decode-residue feature gate of the attention adapter
(ShawRong/ResInfer quant/vllm_integration/attn/runtime.py:1-24)."""
from __future__ import annotations

import os

_QK_RESIDUE = os.environ.get("RESIDUE_ATTN_DISABLE_QK_RESIDUE", "0") != "1"


def _validate_residue_geometry(num_qo_heads: int, num_kv_heads: int) -> None:
    """The serving contract: Q with its residue folded in, query groups of 4, 6 or 8 heads."""
    if not _QK_RESIDUE:
        raise NotImplementedError("ordinary QK is not supported")
    if num_kv_heads <= 0 or num_qo_heads % num_kv_heads or num_qo_heads // num_kv_heads not in (4, 6, 8):
        raise NotImplementedError("production ResAttn requires GQA4/6/8")


def _load_decode_kernel():
    """The host module of the decode kernel.  Loading it opens the shared library, which must exist: there is
    no other implementation behind this adapter."""
    try:
        from ....nvfp4.cute_attn import host
        from .... import _cabi
        _cabi.load()
    except Exception as exc:
        raise RuntimeError("Failed to load ResAttn kernel host resinfer_b200.nvfp4.cute_attn.host") from exc
    return host
