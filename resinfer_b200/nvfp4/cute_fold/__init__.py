"""Fold GEMM (base + residue in one contraction) under the reference's ``nvfp4.cute_fold`` name."""
from .host import kext_kloop_gemm_sm100, mext_fold_gemm
from .tactics import kernel_arch_for_capability

__all__ = ["mext_fold_gemm", "kext_kloop_gemm_sm100", "kernel_arch_for_capability"]
