"""Top-level module name that vLLM's ``vllm.general_plugins`` entry point ``residue_patch`` refers to
(ShawRong/ResInfer runtime/vllm_plugin/pyproject.toml:16-19: ``residue_patch = "residue_vllm_plugin:apply"``)."""
from resinfer_b200.runtime.vllm_plugin.residue_vllm_plugin import apply  # noqa: F401

__all__ = ["apply"]
