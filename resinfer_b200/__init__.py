"""resinfer_b200 -- B200-native kernels for the MEXT / KEXT / ResAttn hot paths of ResInfer.

Layout:
  csrc/ + ../include   CUDA kernels (sm_100a) and the C ABI they are exported through
  _cabi, ops           ctypes binding and tensor-level wrappers
  nvfp4/               the reference's ``nvfp4`` wheel API (quantisers, MXFP4, fold GEMM, ResAttn)
  quant/               linear registry, ``residue::*`` custom ops, tensor-parallel shard plan
  runtime/             the vLLM plugin entry point

``install_aliases()`` makes the package importable under the reference's module names
(``nvfp4``, ``nvfp4.mxfp4``, ``nvfp4.cute_fold``, ``nvfp4.cute_attn``, ``quant``...), so code
written against the reference runs unchanged.
"""
from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"

_ALIASES = {
    "nvfp4": "resinfer_b200.nvfp4",
    "nvfp4.mxfp4": "resinfer_b200.nvfp4.mxfp4",
    "nvfp4.cute_fold": "resinfer_b200.nvfp4.cute_fold",
    "nvfp4.cute_fold.host": "resinfer_b200.nvfp4.cute_fold.host",
    "nvfp4.cute_fold.tactics": "resinfer_b200.nvfp4.cute_fold.tactics",
    "nvfp4.cute_attn": "resinfer_b200.nvfp4.cute_attn",
    "nvfp4.cute_attn.host": "resinfer_b200.nvfp4.cute_attn.host",
    "nvfp4.cute_attn.plan": "resinfer_b200.nvfp4.cute_attn.plan",
    "nvfp4.cute_attn.kv_layout": "resinfer_b200.nvfp4.cute_attn.kv_layout",
    "quant": "resinfer_b200.quant",
    "quant.linear_registry": "resinfer_b200.quant.linear_registry",
    "quant.mxfp4_linear": "resinfer_b200.quant.mxfp4_linear",
    "quant.kernel_metadata": "resinfer_b200.quant.kernel_metadata",
    "quant.vllm_integration": "resinfer_b200.quant.vllm_integration",
    "quant.vllm_integration.residue_linear_op": "resinfer_b200.quant.vllm_integration.residue_linear_op",
    "quant.vllm_integration.residue_tp": "resinfer_b200.quant.vllm_integration.residue_tp",
    "residue_vllm_plugin": "resinfer_b200.runtime.vllm_plugin.residue_vllm_plugin",
}


def install_aliases(overwrite: bool = False) -> list[str]:
    """Register this package under the reference's module names.  Returns the names installed.
    Existing modules of the same name are left alone unless ``overwrite``."""
    done = []
    for alias, target in _ALIASES.items():
        if alias in sys.modules and not overwrite:
            continue
        sys.modules[alias] = importlib.import_module(target)
        done.append(alias)
    return done
