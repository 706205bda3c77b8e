"""Launch selection of the Fold GEMM.

The reference keys a tile shape and a cluster shape on M (csrc/common/fold/sm10x/tactics.py:14-87: tile
(128, 64) on cluster (1, 1) up to 64 tokens, (256, 128) on (2, 1) above) and gates on the architecture
(:22-24, host.py:58-59: only compute capability (10, 0) is served).  This library's kernel has one tile
shape per operand role (128 weight rows x 16..256 token columns, or 256 weight rows on a pair of CTAs), so
what is selected per (M, N, K) is how the (output tile, K tile) units are cut into CTA ranges: whole tiles,
even K slices, ragged ranges over all SMs, or two-CTA tiles.  The selection lives in the library (a table
measured on B200 for the benchmark model's projection shapes, a cost model for everything else);
``describe_plan`` reports it.
"""
from __future__ import annotations


def kernel_arch_for_capability(major: int, minor: int) -> str | None:
    return "sm100" if (major, minor) == (10, 0) else None


def describe_plan(m: int, n: int, k: int, fmt: str = "nvfp4", layout: str = "row_pair") -> dict:
    """What ``fp4_gemm(..., splits=0)`` will launch for this shape on the current device (148 SMs assumed
    when no device is visible): ``k_split`` = 1 for whole tiles, otherwise about how many CTAs share an
    output tile; ``workspace_bytes`` = scratch a K-split plan needs."""
    from ... import _cabi
    lib = _cabi.load()
    fmt_c = {"nvfp4": _cabi.FMT_NVFP4, "mxfp4": _cabi.FMT_MXFP4}[fmt]
    lay_c = {"plain": _cabi.GEMM_PLAIN, "row_pair": _cabi.GEMM_ROW_PAIR, "concat_k": _cabi.GEMM_CONCAT_K}[layout]
    return {"k_split": int(lib.ri_fp4_gemm_auto_splits(m, n, k, fmt_c, lay_c)),
            "workspace_bytes": int(lib.ri_fp4_gemm_workspace_bytes(m, n, k, fmt_c, lay_c, 0))}
