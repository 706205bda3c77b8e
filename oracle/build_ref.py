"""Build recipe for ``oracle/_ref/libnvfp4_ref.so`` (test infrastructure, not product code).

Compiles the reference project's native quantisers from the reference checkout, where the
sources lie, with the flags of the reference's csrc/setup.py:26-76 (``-O3 --use_fast_math``,
``compute_100a/sm_100a``, ``-DENABLE_NVFP4_SM100=1``) plus ``--expt-relaxed-constexpr`` (torch's
BuildExtension adds it).  Nothing is copied: object files and the shared library go to
``oracle/_ref/`` only, which is git-ignored.  The library registers the reference kernels as
torch ops ``nvfp4_ref::*`` (see ref_shim.cpp) and is used by the GPU parity tests as the
bit-exact checker for FP4 codes and block scales.

Usage:  python oracle/build_ref.py [--reference /path/to/ResInfer] [--jobs N]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

REF_SOURCES = [
    "csrc/common/cuda/cuda_utils_kernels.cu",
    "csrc/nvfp4/cuda/nvfp4_quant_entry.cu",
    "csrc/nvfp4/cuda/nvfp4_quant_kernels.cu",
    "csrc/nvfp4/cuda/nvfp4_residue_pack8.cu",
    "csrc/nvfp4/cuda/nvfp4_residue_pack16.cu",
    "csrc/mxfp4/cuda/mxfp4_residue_quant.cu",
]


def default_reference() -> Path:
    """The reference checkout: ``$RESINFER_REFERENCE``, else a directory ``reference`` beside this repository."""
    env = os.environ.get("RESINFER_REFERENCE")
    return Path(env) if env else Path(__file__).resolve().parents[2] / "reference"


def build(reference: Path | None = None, jobs: int = 0, verbose: bool = True) -> Path | None:
    """Return the path of the built library, or None when the reference checkout is absent."""
    reference = Path(reference) if reference else default_reference()
    lib = OUT / "libnvfp4_ref.so"
    if not (reference / "csrc" / "setup.py").exists():
        return lib if lib.exists() else None
    import torch  # noqa: F401  (headers + libs)
    from torch.utils import cpp_extension as ce

    OUT.mkdir(exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")]
    inc += [f"-I{reference / 'csrc/common/cuda'}", f"-I{reference / 'csrc/common/fp4'}"]
    import sysconfig
    inc += [f"-I{sysconfig.get_paths()['include']}"]  # torch/extension.h pulls in Python.h
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    flags = [
        "-std=c++17", "-O3", "-DNDEBUG", "--use_fast_math",
        "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
        "-diag-suppress", "177", "--expt-relaxed-constexpr",
        "-gencode", "arch=compute_100a,code=sm_100a", "-DENABLE_NVFP4_SM100=1",
        "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
        "-Xcompiler", "-fPIC",
    ]
    units = [(reference / s, OUT / (Path(s).stem + ".o")) for s in REF_SOURCES]
    units.append((HERE / "ref_shim.cpp", OUT / "ref_shim.o"))

    def compile_one(unit):
        src, obj = unit
        if obj.exists() and obj.stat().st_mtime >= src.stat().st_mtime:
            return
        cmd = [nvcc, *flags, *inc, "-c", str(src), "-o", str(obj)]
        if verbose:
            print("[build_ref]", src.name, flush=True)
        subprocess.run(cmd, check=True)

    jobs = jobs or min(len(units), os.cpu_count() or 1)
    with ThreadPoolExecutor(jobs) as pool:
        list(pool.map(compile_one, units))

    libdirs = ce.library_paths("cuda")
    link = [nvcc, "-shared", "-o", str(lib), *[str(o) for _, o in units]]
    for d in libdirs:
        link += [f"-L{d}"]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda",
             "-Xlinker", f"-rpath={libdirs[0]}"]
    subprocess.run(link, check=True)
    if verbose:
        print("[build_ref] wrote", lib)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--jobs", type=int, default=0)
    a = ap.parse_args()
    out = build(a.reference, a.jobs)
    if out is None:
        print("reference checkout not found; nothing built", file=sys.stderr)
        sys.exit(1)
