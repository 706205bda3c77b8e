"""Tensor-level entry points of the GEMM and attention kernels (thin wrappers over the C ABI).

These are the functions the reference-named modules (``nvfp4.cute_fold.host``,
``nvfp4.mxfp4.dense``, ``nvfp4.cute_attn.host``) call.  Workspaces are cached per
(device, size) like the reference caches its reduction workspaces
(ShawRong/ResInfer quant/vllm_integration/attn/decode.py:23-53); nothing is allocated once a
shape has been seen, so the calls stay CUDA-graph capturable after a warm-up.

One rule follows from the sharing: calls that use the same cached workspace (same device, same kind,
same size) must not overlap on the GPU -- issue them on one stream, or order the streams with events.
The split tickets in a workspace are left at zero by every launch that completes.
"""
from __future__ import annotations

import contextlib

import torch

from . import _cabi

_WORKSPACES: dict[tuple, torch.Tensor] = {}
_TICKET_BYTES: dict[tuple, int] = {}
_STATUS: dict[torch.device, torch.Tensor] = {}
_GEMM_PLANS: dict[tuple, tuple] = {}


class _on_device:
    """``torch.cuda.device(dev)`` that costs nothing when ``dev`` is already current (the usual case)."""

    __slots__ = ("ctx",)

    def __init__(self, dev):
        self.ctx = None if dev.index is None or torch.cuda.current_device() == dev.index else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)



def _workspace(device, nbytes: int, tag: str, zero_prefix: int = 0) -> torch.Tensor:
    key = (str(device), tag, nbytes)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        if zero_prefix:
            ws[:zero_prefix].zero_()
        _WORKSPACES[key] = ws
        _TICKET_BYTES[key] = int(zero_prefix)
    return ws


def status_word(device) -> torch.Tensor:
    """Device int32 that kernels set non-zero when one of their bounded waits expired."""
    device = torch.device(device)
    st = _STATUS.get(device)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device] = st
    return st


def check_status(device) -> None:
    """Synchronising check of the status word.  A non-zero word means that a bounded device-side wait
    expired in some launch since the last check: that launch's output is invalid and it may have left
    split tickets behind, so the ticket areas of the cached workspaces of the device are cleared before
    the error is raised."""
    st = status_word(device)
    v = int(st.item())
    if v:
        st.zero_()
        for key, ws in _WORKSPACES.items():
            if key[0] == str(torch.device(device)) and _TICKET_BYTES.get(key):
                ws[:_TICKET_BYTES[key]].zero_()
        raise RuntimeError(f"a device-side wait expired (status {v})")


_ACTIVE_REDUCER = None
_ACTIVE_REDUCER_EPILOGUE = True
_NO_REDUCER = object()                   # "no reduction for this call" inside a row_parallel_reduction block


@contextlib.contextmanager
def row_parallel_reduction(reducer, epilogue: bool = True):
    """Inside the block every ``fp4_gemm`` call without an explicit ``allreduce`` argument -- in particular the
    ones made by ``residue::nvfp4_linear`` and ``residue::mxfp4_linear``, whose schemas have no room for it --
    returns its output summed over the ranks of ``reducer`` (a ``resinfer_b200.quant.tp.PeerAllReduce``):
    in the GEMM's epilogue (``epilogue=True``), or by the stand-alone kernel with the GEMM writing its partial
    straight into the exported buffer (``epilogue=False``: two launches, no copy in between).  This is where a
    tensor-parallel model wraps the linear of a row-parallel layer; ``None`` switches it off again for a nested
    block.  Process-wide, not per thread."""
    global _ACTIVE_REDUCER, _ACTIVE_REDUCER_EPILOGUE
    prev = (_ACTIVE_REDUCER, _ACTIVE_REDUCER_EPILOGUE)
    _ACTIVE_REDUCER, _ACTIVE_REDUCER_EPILOGUE = reducer, bool(epilogue)
    try:
        yield reducer
    finally:
        _ACTIVE_REDUCER, _ACTIVE_REDUCER_EPILOGUE = prev


def fp4_gemm(act: torch.Tensor, act_sf: torch.Tensor, weight: torch.Tensor, weight_sf: torch.Tensor,
             alpha: torch.Tensor | None, *, m: int, fmt: str = "nvfp4", layout: str = "plain",
             out_dtype: torch.dtype = torch.bfloat16, out: torch.Tensor | None = None,
             splits: int = 0, enable_pdl: bool = True, allreduce=None) -> torch.Tensor:
    """out[m, N] = alpha * act . weight^T with block-scaled FP4 operands.

    act: uint8 codes, [M, K/2] (plain), [2M, K/2] (row_pair) or [M, K] (concat_k); weight uint8
    [N, K/2] (row stride may exceed K/2); scale buffers 128x4-swizzled uint8 (E4M3 for nvfp4, E8M0
    for mxfp4); alpha float32 device tensor with 1 (or, row_pair, 2) elements or None.

    ``allreduce``: a ``resinfer_b200.quant.tp.PeerAllReduce`` makes this the GEMM of a row-parallel
    linear: the kernel stores this rank's BF16 partial into every rank's inbox and sums the partials of
    all ranks itself (``ri_fp4_gemm_allreduce``); ``out`` (BF16) receives the sum.  Every
    rank of the group must make the same calls in the same order."""
    lib = _cabi.load()
    if allreduce is None and _ACTIVE_REDUCER is not None:
        if _ACTIVE_REDUCER_EPILOGUE:
            allreduce = _ACTIVE_REDUCER
        else:
            # the GEMM writes this rank's partial into the exported buffer, the stand-alone kernel sums the ranks
            red, n_out = _ACTIVE_REDUCER, weight.shape[0]
            if out_dtype != torch.bfloat16 or (out is not None and out.dtype != torch.bfloat16):
                raise ValueError("the all-reduce sums BF16 partials")
            part = fp4_gemm(act, act_sf, weight, weight_sf, alpha, m=m, fmt=fmt, layout=layout, out_dtype=out_dtype,
                            out=red.partial((m, n_out)), splits=splits, enable_pdl=enable_pdl, allreduce=_NO_REDUCER)
            return red.reduce(part, out)
    if allreduce is _NO_REDUCER:
        allreduce = None
    fmt_c = {"nvfp4": _cabi.FMT_NVFP4, "mxfp4": _cabi.FMT_MXFP4}[fmt]
    lay_c = {"plain": _cabi.GEMM_PLAIN, "row_pair": _cabi.GEMM_ROW_PAIR, "concat_k": _cabi.GEMM_CONCAT_K}[layout]
    n, kp = weight.shape
    k = kp * 2
    dev = weight.device
    if weight.stride(1) != 1:
        raise ValueError(f"weight must stay K-contiguous within a row; got stride {weight.stride()}")
    if act.dim() != 2 or act.stride(1) != 1:
        raise ValueError(f"activation must be compact rows; got stride {act.stride()}")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=dev)
    with _on_device(dev):
        ws = None
        plan_key = (dev.index, m, n, k, fmt_c, lay_c, splits)
        plan = _GEMM_PLANS.get(plan_key)
        if plan is None:                                   # workspace size of a shape, asked once per device
            plan = (lib.ri_fp4_gemm_workspace_bytes(m, n, k, fmt_c, lay_c, splits), lib.ri_fp4_gemm_counter_bytes(m, n))
            _GEMM_PLANS[plan_key] = plan
        ws_bytes = plan[0]
        if ws_bytes < 0:
            _cabi.check(_cabi.RI_ERR_ARG, "fp4_gemm plan")
        if ws_bytes > 0:
            ws = _workspace(dev, ws_bytes, "gemm", zero_prefix=plan[1])
        if allreduce is not None:
            if out.dtype != torch.bfloat16 or out.stride(1) != 1:
                raise ValueError("the fused all-reduce writes a BF16 result with contiguous rows")
            inboxes, area = allreduce.next_inbox(m * n)
            st = lib.ri_fp4_gemm_allreduce(
                act.data_ptr(), act.stride(0), act_sf.data_ptr(), act_sf.numel(),
                weight.data_ptr(), weight.stride(0), weight_sf.data_ptr(), weight_sf.numel(),
                _cabi.ptr(alpha), 0 if alpha is None else alpha.numel(), n, m, n, k, fmt_c, lay_c,
                splits, _cabi.ptr(ws), ws_bytes, allreduce.status.data_ptr(), int(enable_pdl),
                _cabi.current_stream(dev), inboxes, area, allreduce.tile_flag_ptrs,
                allreduce.tile_calls.data_ptr(), allreduce.max_tiles, allreduce.rank, allreduce.world,
                out.data_ptr(), out.stride(0))
            _cabi.check(st, "fp4_gemm_allreduce")
            return out
        st = lib.ri_fp4_gemm(
            act.data_ptr(), act.stride(0), act_sf.data_ptr(), act_sf.numel(),
            weight.data_ptr(), weight.stride(0), weight_sf.data_ptr(), weight_sf.numel(),
            _cabi.ptr(alpha), 0 if alpha is None else alpha.numel(),
            out.data_ptr(), _cabi.torch_dtype_code(out.dtype, allow_f32=True), out.stride(0), m, n, k, fmt_c, lay_c,
            splits, _cabi.ptr(ws), ws_bytes, status_word(dev).data_ptr(), int(enable_pdl),
            _cabi.current_stream(dev))
    _cabi.check(st, "fp4_gemm")
    return out


def fp4_gemm_static_scratch(act: torch.Tensor, act_sf: torch.Tensor, weight: torch.Tensor,
                            weight_sf: torch.Tensor, alpha: torch.Tensor | None, *, m: int, out: torch.Tensor,
                            fmt: str = "nvfp4", layout: str = "plain", splits: int = 0,
                            enable_pdl: bool = True) -> torch.Tensor:
    """`fp4_gemm` through the entry point that allocates nothing: `out` is required, the K-split
    scratch is the library's built-in per-device array (shared by all calls on the device, so calls
    must not overlap in time), and sizes that need more than that array raise RuntimeError."""
    lib = _cabi.load()
    fmt_c = {"nvfp4": _cabi.FMT_NVFP4, "mxfp4": _cabi.FMT_MXFP4}[fmt]
    lay_c = {"plain": _cabi.GEMM_PLAIN, "row_pair": _cabi.GEMM_ROW_PAIR, "concat_k": _cabi.GEMM_CONCAT_K}[layout]
    n, kp = weight.shape
    dev = weight.device
    if weight.stride(1) != 1 or act.dim() != 2 or act.stride(1) != 1:
        raise ValueError("operands must be K-contiguous rows")
    with torch.cuda.device(dev):
        st = lib.ri_fp4_gemm_static_scratch(
            act.data_ptr(), act.stride(0), act_sf.data_ptr(), act_sf.numel(),
            weight.data_ptr(), weight.stride(0), weight_sf.data_ptr(), weight_sf.numel(),
            _cabi.ptr(alpha), 0 if alpha is None else alpha.numel(),
            out.data_ptr(), _cabi.torch_dtype_code(out.dtype, allow_f32=True), out.stride(0), m, n, kp * 2,
            fmt_c, lay_c, splits, status_word(dev).data_ptr(), int(enable_pdl), _cabi.current_stream(dev))
    _cabi.check(st, "fp4_gemm_static_scratch")
    return out


@contextlib.contextmanager
def resattn_pv_format(fmt: str):
    """Inside the block ``resattn_decode`` runs its second product in ``fmt``: "fp16" (the default: V exact,
    P with 11 bits) or "e4m3" (V and P rounded to E4M3 like the reference's kernel: faster, about ten times
    further from exact attention).  Process-wide (``ri_resattn_set_pv_format``)."""
    lib = _cabi.load()
    code = {"fp16": 0, "e4m3": 1}[fmt]
    prev = int(lib.ri_resattn_get_pv_format())
    lib.ri_resattn_set_pv_format(code)
    try:
        yield
    finally:
        lib.ri_resattn_set_pv_format(prev)


def kv_page_strides(k_data: torch.Tensor, k_sf: torch.Tensor, v_data: torch.Tensor, v_sf: torch.Tensor):
    """(code bytes, scale bytes) between consecutive pages of a paged NVFP4 KV pool.

    Each of the four tensors is [pages, Hkv, page, D/2 or D/16] with the three inner dimensions dense; the page
    stride is free, so the views vLLM cuts out of its interleaved cache (every page = K codes | K scales |
    V codes | V scales) are taken as they are.  K and V must share their strides."""
    def one(t, name):
        _, h, page, w = t.shape
        want = (page * w, w, 1)
        if t.element_size() != 1 or tuple(t.stride()[1:]) != want or (t.shape[0] > 1 and t.stride(0) < h * page * w):
            raise ValueError(f"{name} must be a byte tensor [pages, Hkv, page, {w}] with dense inner dimensions, got "
                             f"shape {tuple(t.shape)} strides {tuple(t.stride())}")
        return int(t.stride(0)) if t.shape[0] > 1 else h * page * w
    kc, vc = one(k_data, "k_data"), one(v_data, "v_data")
    ks, vs = one(k_sf, "k_sf"), one(v_sf, "v_sf")
    if kc != vc or ks != vs:
        raise ValueError(f"K and V must have the same page strides, got codes {kc} / {vc}, scales {ks} / {vs}")
    return kc, ks


def resattn_decode(q: torch.Tensor, k_data: torch.Tensor, k_sf: torch.Tensor, v_data: torch.Tensor,
                   v_sf: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                   score_scale: float, out_scale: float, out: torch.Tensor, *, splits: int = 1,
                   q_residue: bool = True, q_pack: torch.Tensor | None = None,
                   q_sf: torch.Tensor | None = None, max_kv_len: int = 0,
                   out_global_scale: torch.Tensor | None = None,
                   out_block_scale: torch.Tensor | None = None, reducer: str = "ticket") -> torch.Tensor:
    """Paged NVFP4-KV decode attention.  q bf16 [B,Hq,D]; k_data/v_data uint8 [pages,Hkv,page,D/2];
    k_sf/v_sf uint8 (or float8_e4m3fn) [pages,Hkv,page,D/16] (any page stride: ``kv_page_strides``); out bf16 [B,Hq,D] (written) -- or, with
    ``out_global_scale`` (float32[1]) and ``out_block_scale`` (128x4-swizzled E4M3 bytes), packed NVFP4:
    out uint8 [B, Hq*D/2].  ``reducer``: how the KV splits are combined, "ticket" (through a workspace, the CTA
    that finishes last) or "cluster" (2 to 8 or 16 splits as one thread-block cluster, through shared memory); same bits."""
    lib = _cabi.load()
    b, hq, d = q.shape
    pages, hkv, page, _ = k_data.shape
    dev = q.device
    code_stride, sf_stride = kv_page_strides(k_data, k_sf, v_data, v_sf)
    reducer_c = {"ticket": _cabi.ATTN_REDUCER_TICKET, "cluster": _cabi.ATTN_REDUCER_CLUSTER}[reducer]
    with torch.cuda.device(dev):
        ws = None
        ws_bytes = 0
        if splits > 1 and reducer == "ticket":
            ws_bytes = lib.ri_resattn_workspace_bytes(b, hq, d, splits)
            ws = _workspace(dev, ws_bytes, "attn", zero_prefix=lib.ri_resattn_counter_bytes(b, hq))
        st = lib.ri_resattn_decode_strided(
            q.data_ptr(), k_data.data_ptr(), k_sf.data_ptr(), v_data.data_ptr(), v_sf.data_ptr(), pages,
            code_stride, sf_stride, block_tables.data_ptr(), block_tables.stride(0), seq_lens.data_ptr(), b, hq, hkv, d, page,
            int(max_kv_len), float(score_scale), float(out_scale), out.data_ptr(),
            _cabi.DTYPE_NVFP4 if out_block_scale is not None else _cabi.torch_dtype_code(out.dtype, allow_f32=True),
            _cabi.ptr(q_pack), 0 if q_pack is None else q_pack.numel(),
            _cabi.ptr(q_sf), 0 if q_sf is None else q_sf.numel(),
            _cabi.ptr(out_global_scale), _cabi.ptr(out_block_scale),
            0 if out_block_scale is None else out_block_scale.numel() * out_block_scale.element_size(),
            splits, reducer_c, _cabi.ptr(ws), ws_bytes, int(q_residue), status_word(dev).data_ptr(),
            _cabi.current_stream(dev))
    _cabi.check(st, "resattn_decode")
    return out


def rcp_approx(x: torch.Tensor) -> torch.Tensor:
    """rcp.approx.ftz.f32 of a float32 CUDA tensor (test helper)."""
    lib = _cabi.load()
    x = x.contiguous()
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _cabi.check(lib.ri_rcp_approx(x.data_ptr(), y.data_ptr(), x.numel(), _cabi.current_stream(x.device)),
                    "rcp_approx")
    return y
