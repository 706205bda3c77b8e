"""Registration of ResAttn as vLLM's CUSTOM attention backend
(ShawRong/ResInfer quant/vllm_integration/attn/register.py:17-78): gated by ``RESIDUE_ATTN=1``, refuses to
replace a CUSTOM backend somebody else registered, checks the registry's shape before touching it and reports
every refusal through the diagnostics log instead of raising -- a vLLM without the hook keeps its own attention.
"""
from __future__ import annotations

import inspect
import os

from .. import diagnostics

_INSTALLED_ATTR = "_residue_res_attn_registered"
_BACKEND_CLASS_PATH = "resinfer_b200.quant.vllm_integration.attn.backend.ResAttnFlashInferBackend"


def _registry_shape_ok(reg) -> bool:
    """vLLM's custom-backend API as this module uses it: ``register_backend(backend, class_path)`` and an
    ``AttentionBackendEnum`` with a CUSTOM member."""
    if not hasattr(reg, "register_backend") or not hasattr(reg, "AttentionBackendEnum"):
        diagnostics.log_registration_failure("registry lacks register_backend/AttentionBackendEnum")
        return False
    if "CUSTOM" not in reg.AttentionBackendEnum.__members__:
        diagnostics.log_registration_failure("registry has no CUSTOM member")
        return False
    try:
        params = inspect.signature(reg.register_backend).parameters
    except (TypeError, ValueError) as exc:
        diagnostics.log_registration_failure("cannot introspect register_backend", exc)
        return False
    if "backend" not in params or "class_path" not in params:
        diagnostics.log_registration_failure("register_backend signature changed", list(params))
        return False
    return True


def install(force: bool = False, registry=None) -> bool:
    """Register the backend when ``RESIDUE_ATTN=1`` (or ``force``); True if it is registered afterwards.
    ``registry`` replaces ``vllm.v1.attention.backends.registry`` (tests)."""
    if not force and os.environ.get("RESIDUE_ATTN") != "1":
        return False
    reg = registry
    if reg is None:
        try:
            import vllm.v1.attention.backends.registry as reg
        except Exception as exc:
            diagnostics.log_registration_failure("vLLM attention registry unavailable", exc)
            return False
    if getattr(reg, _INSTALLED_ATTR, False):
        return True
    if not _registry_shape_ok(reg):
        return False
    if reg.AttentionBackendEnum.CUSTOM.is_overridden():
        try:
            other = reg.AttentionBackendEnum.CUSTOM.get_path()
        except Exception:
            other = "<unknown>"
        diagnostics.log_registration_failure("CUSTOM already registered; refusing to overwrite", other)
        return False
    try:
        from vllm.v1.attention.backend import AttentionBackend

        from .backend import ResAttnFlashInferBackend
        if not issubclass(ResAttnFlashInferBackend, AttentionBackend):
            raise TypeError("ResAttnFlashInferBackend is not an AttentionBackend")
    except Exception as exc:
        diagnostics.log_registration_failure("backend class failed to import/validate", exc)
        return False
    reg.register_backend(reg.AttentionBackendEnum.CUSTOM, class_path=_BACKEND_CLASS_PATH)
    setattr(reg, _INSTALLED_ATTR, True)
    diagnostics.log_registration_success(_BACKEND_CLASS_PATH)
    return True
