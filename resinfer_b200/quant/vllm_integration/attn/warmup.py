"""Decode-kernel variants declared to vLLM's warm-up phase
(ShawRong/ResInfer quant/vllm_integration/attn/warmup.py:14-60).

The reference compiles its CuTe-DSL kernel at run time, one specialisation per (geometry, plan), and lists those
compilations here so vLLM runs them before serving.  This library's kernels are compiled into the shared library
ahead of time; a "compile unit" here loads the library and sets the instantiation's launch attributes, so the
first request pays nothing.  The provider is handed to vLLM when its CuTe-DSL warm-up registry exists
(``vllm.model_executor.warmup.cutedsl_warmup``, vLLM 0.26); on older vLLM it is kept for ``warm_now``.
"""
from __future__ import annotations

import functools
from typing import NamedTuple

import torch

from .runtime import _load_decode_kernel, _validate_residue_geometry


class _Unit(NamedTuple):
    """Stand-in for vLLM's ``CuTeDSLCompileUnit`` where that class does not exist: same three fields."""
    name: str
    key: tuple
    compile: object


def _unit_cls():
    try:
        from vllm.model_executor.warmup.cutedsl_warmup import CuTeDSLCompileUnit
        return CuTeDSLCompileUnit
    except Exception:
        return _Unit


class _DecodeWarmupProvider:
    """Variants only: no model forward, no timing, no KV pages."""

    def __init__(self):
        self._geometries: set[tuple[int, int, int, bool]] = set()

    def add_geometry(self, num_qo_heads, num_kv_heads, head_dim, fuse_attn_quant):
        self._geometries.add((int(num_qo_heads), int(num_kv_heads), int(head_dim), bool(fuse_attn_quant)))

    def get_cutedsl_warmup_compile_units(self):
        if not torch.cuda.is_available():
            return []
        host = _load_decode_kernel()
        unit = _unit_cls()
        units, seen = [], set()
        for hq, hkv, dim, packed in sorted(self._geometries):
            _validate_residue_geometry(hq, hkv)
            for output_nvfp4 in ((False, True) if packed else (False,)):
                for spec in host.decode_compile_variants(hq, hkv, dim, residue_fold=True, output_nvfp4=output_nvfp4):
                    key = ("resattn_decode", spec["args"], tuple(sorted(spec["kwargs"].items())))
                    if key in seen:
                        continue
                    seen.add(key)
                    units.append(unit(name=f"resattn_decode[{spec['label']}]", key=key,
                                      compile=functools.partial(host.compile_decode_variant, spec)))
        return units

    def warm_now(self) -> int:
        """Run every unit; the number run."""
        units = self.get_cutedsl_warmup_compile_units()
        for u in units:
            u.compile()
        return len(units)


# vLLM keeps providers in a WeakSet: this reference keeps the provider alive for the worker's lifetime
_DECODE_WARMUP_PROVIDER: _DecodeWarmupProvider | None = None


def _fuse_attn_quant_enabled() -> bool:
    try:
        from vllm.config import get_current_vllm_config_or_none
        cfg = get_current_vllm_config_or_none()
        return bool(cfg is not None and cfg.compilation_config is not None
                    and cfg.compilation_config.pass_config.fuse_attn_quant)
    except Exception:
        return False


def _register_decode_warmup(num_qo_heads, num_kv_heads, head_dim) -> _DecodeWarmupProvider:
    global _DECODE_WARMUP_PROVIDER
    packed = bool(head_dim == 128 and _fuse_attn_quant_enabled())
    if _DECODE_WARMUP_PROVIDER is None:
        _DECODE_WARMUP_PROVIDER = _DecodeWarmupProvider()
    _DECODE_WARMUP_PROVIDER.add_geometry(num_qo_heads, num_kv_heads, head_dim, packed)
    try:
        from vllm.model_executor.warmup.cutedsl_warmup import register_cutedsl_warmup_provider
    except Exception:
        return _DECODE_WARMUP_PROVIDER
    register_cutedsl_warmup_provider(_DECODE_WARMUP_PROVIDER)
    return _DECODE_WARMUP_PROVIDER
