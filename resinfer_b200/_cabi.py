"""ctypes binding of ``libresinfer_b200.so`` (the C ABI declared in ``include/resinfer_b200.h``).

There is no CPU fallback: if the shared library is missing or a call is rejected the caller
gets an exception (``ImportError`` / ``RuntimeError`` / ``NotImplementedError``), mirroring the
``TORCH_CHECK`` / ``TORCH_CHECK_NOT_IMPLEMENTED`` behaviour of the reference's native ops
(ShawRong/ResInfer csrc/nvfp4/cuda/nvfp4_quant_entry.cu:183-185).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "_lib" / "libresinfer_b200.so"

RI_ERR_ARG, RI_ERR_UNSUPPORTED, RI_ERR_DEVICE, RI_ERR_TIMEOUT = -1, -2, -3, -4
DTYPE_BF16, DTYPE_FP16, DTYPE_F32, DTYPE_NVFP4 = 0, 1, 2, 3
ATTN_REDUCER_TICKET, ATTN_REDUCER_CLUSTER = 0, 1
FMT_NVFP4, FMT_MXFP4 = 0, 1
GEMM_PLAIN, GEMM_ROW_PAIR, GEMM_CONCAT_K = 0, 1, 2

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "ri_abi_version": (_i, []),
    "ri_last_error": (C.c_char_p, []),
    "ri_device_info": (_i, [C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "ri_nvfp4_quant_mext": (_i, [_vp, _i, _i, _i, _i64, _vp, _i, _vp, _i64, _vp, _i64, _i, _i, _vp]),
    "ri_nvfp4_quant_kext": (_i, [_vp, _i, _i, _i, _i64, _vp, _vp, _i, _i, _vp, _i64, _vp, _i64, _i, _vp]),
    "ri_nvfp4_quant_grouped_q": (_i, [_vp, _i, _i, _i, _i, _vp, _i64, _vp, _i64, _vp]),
    "ri_mxfp4_quant": (_i, [_vp, _i, _i, _i, _i64, _i64, _vp, _i, _vp, _i, _i, _vp, _i64, _i, _i, _i, _vp]),
    "ri_fp4_gemm": (_i, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i, _vp, _i, _i64, _i, _i, _i,
                         _i, _i, _i, _vp, _i64, _vp, _i, _vp]),
    "ri_fp4_gemm_static_scratch": (_i, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i, _vp, _i, _i64, _i, _i,
                                        _i, _i, _i, _i, _vp, _i, _vp]),
    "ri_fp4_gemm_workspace_bytes": (_i64, [_i, _i, _i, _i, _i, _i]),
    "ri_fp4_gemm_counter_bytes": (_i64, [_i, _i]),
    "ri_fp4_gemm_auto_splits": (_i, [_i, _i, _i, _i, _i]),
    "ri_fp4_gemm_allreduce_tiles": (_i64, [_i, _i]),
    "ri_fp4_gemm_allreduce_uses_pairs": (_i, [_i, _i, _i]),
    "ri_fp4_gemm_allreduce_flag_bytes": (_i64, [_i64]),
    "ri_fp4_gemm_allreduce_call_bytes": (_i64, [_i64]),
    "ri_fp4_gemm_allreduce": (_i, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i, _i64, _i, _i, _i, _i, _i, _i,
                                   _vp, _i64, _vp, _i, _vp, _vp, _i64, _vp, _vp, _i64, _i, _i, _vp, _i64]),
    "ri_resattn_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i, _i, _i, _i, _i, _i, _f, _f,
                               _vp, _i, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i, _vp, _i64, _i, _vp, _vp]),
    "ri_resattn_decode_strided": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _i, _i, _i, _i, _i, _i,
                                       _f, _f, _vp, _i, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i, _i, _vp, _i64, _i, _vp, _vp]),
    "ri_resattn_prepare": (_i, [_i]),
    "ri_resattn_workspace_bytes": (_i64, [_i, _i, _i, _i]),
    "ri_resattn_counter_bytes": (_i64, [_i, _i]),
    "ri_resattn_set_pv_format": (None, [_i]),
    "ri_resattn_get_pv_format": (_i, []),
    "ri_peer_allreduce_flag_bytes": (_i64, []),
    "ri_peer_allreduce_state_bytes": (_i64, []),
    "ri_peer_allreduce_set_wait_ms": (None, [_i]),
    "ri_peer_allreduce_bf16": (_i, [_vp, _vp, _i, _i, _i64, _vp, _vp, _vp, _vp, _i]),
    "ri_rcp_approx": (_i, [_vp, _vp, _i, _vp]),
}

_lib = None


def load(build_if_missing: bool | None = None) -> C.CDLL:
    """Load the shared library (once).  Set RESINFER_B200_AUTOBUILD=1 (or pass
    ``build_if_missing=True``) to compile it first when it is absent or older than its sources."""
    global _lib
    if _lib is not None:
        return _lib
    if build_if_missing is None:
        build_if_missing = os.environ.get("RESINFER_B200_AUTOBUILD", "0") == "1"
    if build_if_missing:
        from . import build as _build
        _build.build()
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} not found. Build it with `python -m resinfer_b200.build` "
            "(needs nvcc; compiles for sm_100a). There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)            # AttributeError = stale binary: fail loudly
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().ri_last_error().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    """Turn a C-ABI status into the exception the reference's op would raise."""
    if status == 0:
        return
    msg = last_error()
    if status in (RI_ERR_UNSUPPORTED, RI_ERR_DEVICE):
        raise NotImplementedError(f"{what}: {msg}")
    if status < 0:
        raise RuntimeError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: CUDA error {status}: {msg}")


def ptr(t) -> int | None:
    """Device pointer of a torch tensor (None stays NULL)."""
    return None if t is None else t.data_ptr()


def current_stream(device) -> int:
    import torch
    return torch.cuda.current_stream(device).cuda_stream


def torch_dtype_code(dtype, allow_f32: bool = False) -> int:
    import torch
    if dtype == torch.bfloat16:
        return DTYPE_BF16
    if dtype == torch.float16:
        return DTYPE_FP16
    if dtype == torch.float32 and allow_f32:
        return DTYPE_F32
    raise RuntimeError("Unsupported input data type for quantize_to_fp4.")
