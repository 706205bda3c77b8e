"""Architecture gate of the Fold GEMM (reference: csrc/common/fold/sm10x/tactics.py:22-24,
host.py:58-59: only compute capability (10, 0) is served)."""
from __future__ import annotations


def kernel_arch_for_capability(major: int, minor: int) -> str | None:
    return "sm100" if (major, minor) == (10, 0) else None
