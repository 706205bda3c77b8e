"""In-tree build of ``libresinfer_b200.so`` with plain nvcc (no torch headers needed).

    python -m resinfer_b200.build [--force] [--verbose]

Every translation unit is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``) and linked into
``resinfer_b200/_lib/libresinfer_b200.so``; the CUDA runtime is linked statically and the driver
API entry point needed for TMA descriptors is resolved at run time, so the library loads (and
exports all its symbols) on a machine without a GPU driver.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OUT_DIR = PKG / "_lib"
LIB = OUT_DIR / "libresinfer_b200.so"

SOURCES = ["api.cu", "quant_nvfp4.cu", "quant_mxfp4.cu", "gemm_fp4.cu", "gemm_static_scratch.cu", "resattn.cu", "peer_allreduce.cu"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr", "-diag-suppress", "177",
]


def _nvcc() -> str:
    return os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    newest_hdr = max((h.stat().st_mtime for h in headers), default=0.0)
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(src: Path) -> Path:
        obj = OUT_DIR / (src.stem + ".o")
        if (not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime
                and obj.stat().st_mtime > newest_hdr):
            return obj
        cmd = [_nvcc(), *flags, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or (ptxas_info and r.stderr):
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    srcs = sources()
    with ThreadPoolExecutor(min(len(srcs), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / smem per kernel")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.ptxas_info))
