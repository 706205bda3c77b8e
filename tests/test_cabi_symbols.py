"""The C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "resinfer_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ri_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from resinfer_b200 import _cabi, build
    build.build()                      # nvcc cross-compiles for sm_100a; no GPU needed
    return _cabi.load()


def test_header_and_binding_agree(lib):
    from resinfer_b200 import _cabi
    names = _declared()
    assert len(names) >= 12
    assert set(names) == set(_cabi.SIGNATURES), set(names) ^ set(_cabi.SIGNATURES)
    for n in names:
        assert getattr(lib, n) is not None


def test_abi_version_and_error_text(lib):
    assert lib.ri_abi_version() == 1
    assert isinstance(lib.ri_last_error(), bytes)


def test_argument_validation_needs_no_gpu(lib):
    """Rejected arguments return RI_ERR_ARG before any CUDA call, with the reference's message."""
    from resinfer_b200 import _cabi
    st = lib.ri_nvfp4_quant_mext(None, 0, 4, 24, 24, None, 1, None, 0, None, 0, 1, 0, None)
    assert st == _cabi.RI_ERR_ARG and b"multiple of 16" in lib.ri_last_error()
    st = lib.ri_nvfp4_quant_kext(None, 0, 4, 256, 256, None, None, 8, 512, None, 0, None, 0, 0, None)
    assert st == _cabi.RI_ERR_ARG and b"no longer supported" in lib.ri_last_error()
    st = lib.ri_mxfp4_quant(None, 0, 4, 48, 48, 1, None, 0, None, 8, 24, None, 0, 1, 0, 0, None)
    assert st == _cabi.RI_ERR_ARG and b"invalid MXFP4 extent" in lib.ri_last_error()
    st = lib.ri_nvfp4_quant_grouped_q(None, 1, 1, 5, 128, None, 0, None, 0, None)
    assert st == _cabi.RI_ERR_ARG and b"GQA4/6/8" in lib.ri_last_error()
    st = lib.ri_fp4_gemm(None, 0, None, 0, None, 0, None, 0, None, 0, None, 0, 0, 4, 128, 100, 0, 0, 1, None, 0, None, 0, None)
    assert st == _cabi.RI_ERR_ARG and b"multiple of 64" in lib.ri_last_error()
    assert lib.ri_resattn_counter_bytes(2, 64) == 512
    assert lib.ri_resattn_workspace_bytes(2, 64, 128, 4) == 512 + 4 * 2 * 64 * (128 + 2) * 4
    assert lib.ri_fp4_gemm_workspace_bytes(16, 5120, 8192, 0, 1, 1) == 0
    assert lib.ri_fp4_gemm_workspace_bytes(16, 5120, 8192, 0, 1, 4) > 4 * 40 * 128 * 32 * 4
    st = lib.ri_peer_allreduce_bf16(None, None, 0, 1, 64, None, None, None, None, 0)
    assert st == _cabi.RI_ERR_ARG and b"2..8 ranks" in lib.ri_last_error()
    st = lib.ri_peer_allreduce_bf16(None, None, 1, 2, 12, None, None, None, None, 0)
    assert st == _cabi.RI_ERR_ARG and b"multiple of 8" in lib.ri_last_error()
    assert lib.ri_peer_allreduce_flag_bytes() == 64 and lib.ri_peer_allreduce_state_bytes() == 16


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from resinfer_b200 import _cabi
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError, match="no CPU fallback"):
        _cabi.load(build_if_missing=False)
