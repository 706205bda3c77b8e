"""vLLM general-plugin entry point (group ``vllm.general_plugins``, name ``residue_patch``).

Same gates and fail-closed behaviour as the reference's
runtime/vllm_plugin/residue_vllm_plugin.py:9-46: nothing happens unless RESIDUE_NVFP4, RESIDUE_MXFP4
or RESIDUE_ATTN is "1"; when a gate is set and anything fails, the exception is re-raised so the
worker refuses to serve without the residue kernels.

What is installed: the native library is loaded and the ``nvfp4::*`` / ``residue::*`` ops are
registered, this package is aliased under the reference's module names, and -- for RESIDUE_NVFP4 --
this library's NVFP4 linear method is patched into vLLM's ModelOpt loader
(``quant/vllm_integration/patch.py``); for RESIDUE_MXFP4 the ``modelopt_mxfp4`` quantisation config and
its linear method are registered (``quant/vllm_integration/linear_method_mxfp4.py``); for RESIDUE_ATTN this
library's attention backend is registered as vLLM's CUSTOM backend
(``quant/vllm_integration/attn/register.py``).
"""
from __future__ import annotations

import os


def initialize() -> None:
    """Install the enabled integrations in the current process."""
    nvfp4 = os.environ.get("RESIDUE_NVFP4") == "1"
    resattn = os.environ.get("RESIDUE_ATTN") == "1"
    mxfp4 = os.environ.get("RESIDUE_MXFP4") == "1"
    if not (nvfp4 or resattn or mxfp4):
        return
    pid = os.getpid()
    try:
        import resinfer_b200
        from resinfer_b200.nvfp4.extension import ensure_loaded
        ensure_loaded(required=True)
        resinfer_b200.install_aliases()
        if mxfp4:
            from resinfer_b200.quant import mxfp4_linear  # noqa: F401
            # registers the "modelopt_mxfp4" quantisation config with vLLM
            from resinfer_b200.quant.vllm_integration import linear_method_mxfp4  # noqa: F401
        if nvfp4:
            from resinfer_b200.quant.vllm_integration import env_contract, residue_linear_op  # noqa: F401
            env_contract.settings()
            # this library's own linear method (resinfer_b200/quant/vllm_integration/linear_method_v2.py)
            from resinfer_b200.quant.vllm_integration import patch
            patch.patch_vllm_modelopt(model_dir=os.environ.get("RESIDUE_VLLM_MODEL_DIR"))
        if resattn:
            from resinfer_b200.quant.vllm_integration.attn.register import install
            if not install():
                raise RuntimeError("ResAttn backend registration was refused")
        print(f"[residue:plugin] applied in pid={pid}", flush=True)
    except Exception as exc:
        print(f"[residue:plugin] FAILED in pid={pid}: {type(exc).__name__}: {exc}\n"
              f"[residue:plugin] refusing to serve without the residue kernels (a residue/ResAttn gate "
              f"was set). Unset the gate to run plain vLLM deliberately.", flush=True)
        raise


def apply() -> None:
    """Stable ``vllm.general_plugins`` entry point, called in every worker."""
    initialize()
