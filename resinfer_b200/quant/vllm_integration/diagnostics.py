"""Log lines of the vLLM adapters (ShawRong/ResInfer quant/vllm_integration/diagnostics.py:84-92 for the
attention-backend registration); logging only, no behaviour."""
from __future__ import annotations

import logging


def _logger():
    return logging.getLogger("resinfer_b200.vllm_integration")


def log_registration_failure(reason: str, detail=None) -> None:
    _logger().warning("ResAttn backend not registered: %s%s", reason, "" if detail is None else f" ({detail})")


def log_registration_success(class_path: str) -> None:
    _logger().info("ResAttn registered as vLLM's CUSTOM attention backend: %s", class_path)
