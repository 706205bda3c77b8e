"""Prepare and launch paged NVFP4 decode attention (ResAttn).

Public functions keep the names, argument order and validation messages of the reference's
csrc/resattn/host.py (``run_paged_fp4_decode_qmul4_tmem`` :489-606, ``plan_qmul4_decode`` :83-92,
``allocate_qmul4_reduction_workspace`` :126-153, ``check_shape_supported`` :64-77).  Differences that
follow from this library's kernel:
  * any page size that is a multiple of 16 is accepted (``pool.page_size``), not only 128;
  * the query quantisation (NVFP4 + NVFP4 residue) is fused into the decode kernel, so there is no
    separate quantiser launch and no cached Q scratch;
  * there is one reducer, fused into the decode launch (the CTA that finishes last merges the partials in
    split order); a caller-supplied reduction workspace is validated like the reference does, the
    partial (o, l, m) buffers themselves live in this library's cached workspace.
"""
from __future__ import annotations

import functools
from typing import Tuple

import torch

from ... import _cabi, ops
from .kv_layout import PAGE_SIZE, SF_VEC, NvFp4PagedKVPool
from .plan import select_decode_plan, static_compile_plans, validate_decode_plan  # noqa: F401

N_PAD = 128
Qmul4ReductionWorkspace = Tuple[torch.Tensor, torch.Tensor, torch.Tensor]
RESIDUE_GQA_GROUPS = (4, 6, 8)


def _residue_padded_group_size(num_qo_heads: int, num_kv_heads: int) -> int:
    """Physical base+residue rows per KV head of the reference's Q tile (8 for GQA4, else 16)."""
    if num_kv_heads <= 0 or num_qo_heads % num_kv_heads:
        raise ValueError("Q heads must be divisible by KV heads")
    g = num_qo_heads // num_kv_heads
    if g == 4:
        return 8
    if g in (6, 8):
        return 16
    raise NotImplementedError(f"residue Q supports logical GQA ratios {RESIDUE_GQA_GROUPS}, got {g}")


def check_shape_supported(num_qo_heads: int, num_kv_heads: int, head_dim: int, prediction: int = 1) -> None:
    """Reject unsupported shapes before launching."""
    if num_kv_heads <= 0 or num_qo_heads % num_kv_heads:
        raise ValueError(f"num_qo_heads({num_qo_heads}) must be a multiple of num_kv_heads({num_kv_heads})")
    if head_dim not in (128, 256):
        raise NotImplementedError(f"ResAttn supports head_dim=128 or 256, got {head_dim}")
    _residue_padded_group_size(num_qo_heads, num_kv_heads)
    if prediction != 1:
        raise NotImplementedError("production ResAttn supports single-token decode only")


@functools.lru_cache(maxsize=8)
def _sm_count(device_str: str) -> int:
    return torch.cuda.get_device_properties(device_str).multi_processor_count


def plan_qmul4_decode(batch, num_kv_heads, max_kv_len, device, *, grouped_head_tile=16, residue_fold=True,
                      head_dim=128, seq_lens=None):
    """(splits, reducer) for a BF16-output decode launch; ``seq_lens``: host lengths, if the caller has them."""
    if not residue_fold:
        raise NotImplementedError("ordinary QK is not supported")
    return select_decode_plan(batch, num_kv_heads, max_kv_len, _sm_count(str(device)),
                              grouped_head_tile=grouped_head_tile, residue_fold=residue_fold, head_dim=head_dim,
                              seq_lens=seq_lens)


def allocate_qmul4_reduction_workspace(splits: int, batch: int, num_qo_heads: int, head_dim: int, device, *,
                                       partial_o_dtype: torch.dtype = torch.float32) -> Qmul4ReductionWorkspace:
    """Allocate split-KV partial buffers: o [S,B,1,H,D], l and m [S,B,1,H] (FP32)."""
    if partial_o_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"partial_o_dtype must be torch.float32 or torch.bfloat16, got {partial_o_dtype}")
    if partial_o_dtype != torch.float32:
        raise NotImplementedError("this library keeps split partials in FP32")
    o = torch.empty(splits, batch, 1, num_qo_heads, head_dim, dtype=torch.float32, device=device)
    l = torch.empty(splits, batch, 1, num_qo_heads, dtype=torch.float32, device=device)
    return o, l, torch.empty_like(l)


def _check_decode_metadata(block_tables, seq_lens, batch, device):
    if (block_tables.dtype != torch.int32 or block_tables.device != device or block_tables.ndim != 2
            or block_tables.shape[0] != batch or block_tables.shape[1] < 1 or block_tables.stride(1) != 1
            or block_tables.stride(0) < block_tables.shape[1]):
        raise ValueError("block_tables must be int32 [batch, max_pages_per_seq] on the Q device, with unit "
                         "column stride and non-overlapping rows")
    if (seq_lens.dtype != torch.int32 or seq_lens.device != device or tuple(seq_lens.shape) != (batch,)
            or not seq_lens.is_contiguous()):
        raise ValueError("seq_lens must be contiguous int32 [batch] on the Q device")


def run_paged_fp4_decode_qmul4_tmem(q: torch.Tensor, pool: NvFp4PagedKVPool, v_data_hnd: torch.Tensor,
                                    v_sf_bthd: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                                    sm_scale: float, out: torch.Tensor, max_seq_len: int = 0,
                                    k_sf_mode: str = "linear", value_scale: float = 1.0,
                                    reduction_workspace: Qmul4ReductionWorkspace | None = None,
                                    residue_fold: bool = True, direct_output: bool = True,
                                    plan: tuple[int, str] | None = None) -> torch.Tensor:
    """Run paged NVFP4 attention with BF16 output.

    ``sm_scale`` already includes the K global scale and ``value_scale`` is the V global scale, as in
    the reference's call sites (quant/vllm_integration/attn/decode.py:92, 158)."""
    if not residue_fold:
        raise NotImplementedError("ordinary QK is not supported")
    if k_sf_mode != "linear":
        raise NotImplementedError("production ResAttn uses linear K scales")
    if direct_output is False:
        raise NotImplementedError("padded output is not supported")
    b, hq, d = q.shape
    h = pool.num_kv_heads
    page = pool.page_size
    check_shape_supported(hq, h, d, prediction=1)
    _check_decode_metadata(block_tables, seq_lens, b, q.device)
    if v_data_hnd.shape != (pool.k_data.shape[0], h, page, d // 2):
        raise ValueError(f"v_data_hnd must be [page, head, {page}, D/2], got {tuple(v_data_hnd.shape)}")
    if v_sf_bthd.shape != (pool.k_data.shape[0], h, page, d // SF_VEC):
        raise ValueError(f"v_sf_bthd must be [page, head, {page}, D/16] (trtllm contract), got "
                         f"{tuple(v_sf_bthd.shape)}")
    if (tuple(out.shape) != (b, hq, d) or out.dtype != torch.bfloat16 or out.device != q.device
            or not out.is_contiguous()):
        raise ValueError("direct_output requires contiguous BF16 [B, H_q, D]")
    if q.dtype != torch.bfloat16 or not q.is_contiguous():
        raise ValueError("q must be contiguous CUDA BF16 [B, H_q, D]")
    if plan is None:
        max_len = max_seq_len or int(seq_lens.max().item())
        splits, reduction = plan_qmul4_decode(b, h, max_len, q.device, head_dim=d,
                                              grouped_head_tile=_residue_padded_group_size(hq, h))
    else:
        validate_decode_plan(plan, head_dim=d)
        splits, reduction = plan
    # "kernel" / "gmem_fused": the ticket merge through the workspace; "cga_sharded": the splits as one cluster
    cluster = reduction == "cga_sharded" and splits > 1
    lib = _cabi.load()
    ws_ptr, ws_bytes = None, 0
    if splits > 1 and not cluster:
        need = lib.ri_resattn_workspace_bytes(b, hq, d, splits)
        if reduction_workspace is not None:
            o_p, l_p, m_p = reduction_workspace
            g_pad = _residue_padded_group_size(hq, h)
            for name, t, shapes in (("o_partial", o_p, ((splits, b, 1, h * g_pad, d), (splits, b, 1, hq, d))),
                                    ("l_partial", l_p, ((splits, b, 1, h * g_pad), (splits, b, 1, hq))),
                                    ("m_partial", m_p, ((splits, b, 1, h * g_pad), (splits, b, 1, hq)))):
                if (tuple(t.shape) not in shapes or t.dtype != torch.float32 or t.device != q.device
                        or not t.is_contiguous()):
                    raise ValueError(f"{name} must be contiguous with dtype in ({torch.float32},), shape "
                                     f"{shapes[0]}, on {q.device}, got shape={tuple(t.shape)} dtype={t.dtype} "
                                     f"device={t.device}")
        ws = ops._workspace(q.device, need, "attn", zero_prefix=lib.ri_resattn_counter_bytes(b, hq))
        ws_ptr, ws_bytes = ws.data_ptr(), need
    code_stride, sf_stride = ops.kv_page_strides(pool.k_data, pool.k_sf, v_data_hnd, v_sf_bthd)
    with torch.cuda.device(q.device):
        st = lib.ri_resattn_decode_strided(
            q.data_ptr(), pool.k_data.data_ptr(), pool.k_sf.data_ptr(), v_data_hnd.data_ptr(),
            v_sf_bthd.data_ptr(), pool.k_data.shape[0], code_stride, sf_stride, block_tables.data_ptr(), block_tables.stride(0),
            seq_lens.data_ptr(), b, hq, h, d, page, int(max_seq_len or 0), float(sm_scale), float(value_scale),
            out.data_ptr(),
            _cabi.DTYPE_BF16, None, 0, None, 0, None, None, 0, splits,
            _cabi.ATTN_REDUCER_CLUSTER if cluster else _cabi.ATTN_REDUCER_TICKET, ws_ptr, ws_bytes, 1,
            ops.status_word(q.device).data_ptr(), _cabi.current_stream(q.device))
    _cabi.check(st, "run_paged_fp4_decode_qmul4_tmem")
    return out


def decode_compile_variants(num_qo_heads, num_kv_heads, head_dim, *, residue_fold, output_nvfp4):
    """The kernel specialisations a (geometry, output format) can launch, as dicts with ``args``, ``kwargs`` and
    ``label`` like the reference's list (csrc/resattn/host.py:635-652).  The reference has one per static plan;
    here the split count, the reducer and the output format are launch arguments of one instantiation per
    head_dim, so the list has one entry."""
    if not residue_fold:
        raise NotImplementedError("ordinary QK is not supported")
    check_shape_supported(num_qo_heads, num_kv_heads, head_dim)
    static_compile_plans(output_nvfp4=output_nvfp4, residue_fold=residue_fold, head_dim=head_dim,
                         grouped_head_tile=_residue_padded_group_size(num_qo_heads, num_kv_heads))
    return [dict(args=(int(head_dim),), kwargs={}, label=f"D{head_dim}")]


def compile_decode_variant(plan: dict):
    """Make one entry of ``decode_compile_variants`` ready to launch on the current device (nothing is compiled:
    the shared library holds the kernel; its launch attributes are set)."""
    lib = _cabi.load()
    _cabi.check(lib.ri_resattn_prepare(*plan["args"]), "compile_decode_variant")
    return plan["args"]


def plan_qmul4_decode_nvfp4(batch, num_qo_heads, num_kv_heads, max_kv_len, device, *, residue_fold=True, seq_lens=None):
    """(splits, reducer) for a packed-NVFP4-output decode launch (head_dim 128 only, as in the reference:
    csrc/resattn/host.py:94-106)."""
    if not residue_fold:
        raise NotImplementedError("ordinary QK is not supported")
    return select_decode_plan(batch, num_kv_heads, max_kv_len, _sm_count(str(device)), output_nvfp4=True,
                              grouped_head_tile=_residue_padded_group_size(num_qo_heads, num_kv_heads),
                              residue_fold=residue_fold, seq_lens=seq_lens)


def allocate_nvfp4_attention_output(batch: int, num_qo_heads: int, head_dim: int, device):
    """Packed output [B, Hq*D/2] uint8 and its 128x4-swizzled E4M3 block scales, viewed
    [ceil(B/128)*128, ceil(Hq*D/16 / 4)*4] like the reference's buffers."""
    hidden = num_qo_heads * head_dim
    out = torch.empty(batch, hidden // 2, dtype=torch.uint8, device=device)
    sf = torch.zeros(((batch + 127) // 128) * 128, ((hidden // SF_VEC + 3) // 4) * 4, dtype=torch.float8_e4m3fn,
                     device=device)
    return out, sf


def run_paged_fp4_decode_qmul4_tmem_nvfp4(q: torch.Tensor, pool: NvFp4PagedKVPool, v_data_hnd: torch.Tensor,
                                          v_sf_bthd: torch.Tensor, block_tables: torch.Tensor,
                                          seq_lens: torch.Tensor, sm_scale: float,
                                          output_global_scale_inv: torch.Tensor, *, out: torch.Tensor | None = None,
                                          output_block_scale: torch.Tensor | None = None, max_seq_len: int = 0,
                                          k_sf_mode: str = "linear", value_scale: float = 1.0,
                                          reduction_workspace: Qmul4ReductionWorkspace | None = None,
                                          plan: tuple[int, str] | None = None, residue_fold: bool = True):
    """Paged attention with the output quantised to NVFP4 in the kernel (the activation format of the
    projection that follows).  Arguments, buffer shapes and errors follow the reference's
    csrc/resattn/host.py:660-760; returns ``(out, output_block_scale)``."""
    if not residue_fold:
        raise NotImplementedError("ordinary QK is not supported")
    if k_sf_mode != "linear":
        raise NotImplementedError("production ResAttn uses linear K scales")
    if q.ndim != 3 or q.dtype != torch.bfloat16 or not q.is_cuda:
        raise ValueError("q must be CUDA BF16 [B, H_q, D]")
    b, hq, d = q.shape
    h = pool.num_kv_heads
    if hq % h:
        raise ValueError(f"H_q={hq} must be divisible by H_kv={h}")
    page = pool.page_size
    check_shape_supported(hq, h, d, prediction=1)
    _check_decode_metadata(block_tables, seq_lens, b, q.device)
    if v_data_hnd.shape != (pool.k_data.shape[0], h, page, d // 2):
        raise ValueError(f"v_data_hnd must be [page, head, {page}, D/2], got {tuple(v_data_hnd.shape)}")
    if v_sf_bthd.shape != (pool.k_data.shape[0], h, page, d // SF_VEC):
        raise ValueError(f"v_sf_bthd must be [page, head, {page}, D/16], got {tuple(v_sf_bthd.shape)}")
    gsi = output_global_scale_inv
    if gsi.device != q.device or gsi.dtype != torch.float32 or gsi.numel() != 1:
        raise ValueError("output_global_scale_inv must be a one-element CUDA float32 tensor")
    if out is None or output_block_scale is None:
        if out is not None or output_block_scale is not None:
            raise ValueError("out and output_block_scale must be supplied together")
        out, output_block_scale = allocate_nvfp4_attention_output(b, hq, d, q.device)
    want_out = (b, hq * d // 2)
    want_sf = (((b + 127) // 128) * 128, ((hq * d // SF_VEC + 3) // 4) * 4)
    if tuple(out.shape) != want_out or out.dtype != torch.uint8 or out.device != q.device or not out.is_contiguous():
        raise ValueError(f"out must be contiguous uint8 {want_out} on {q.device}")
    if (tuple(output_block_scale.shape) != want_sf or output_block_scale.dtype != torch.float8_e4m3fn
            or output_block_scale.device != q.device or not output_block_scale.is_contiguous()):
        raise ValueError(f"output_block_scale must be contiguous E4M3 {want_sf} on {q.device}")
    if plan is None:
        max_len = max_seq_len or int(seq_lens.max().item())
        splits, reduction = plan_qmul4_decode_nvfp4(b, hq, h, max_len, q.device, residue_fold=residue_fold)
    else:
        validate_decode_plan(plan, output_nvfp4=True, head_dim=d)
        splits, reduction = plan
    del reduction, reduction_workspace                # one reducer (fused into the decode launch) with its own cached workspace
    ops.resattn_decode(q, pool.k_data, pool.k_sf, v_data_hnd, v_sf_bthd, block_tables, seq_lens, float(sm_scale),
                       float(value_scale), out, splits=splits, max_kv_len=int(max_seq_len or 0),
                       out_global_scale=gsi, out_block_scale=output_block_scale)
    return out, output_block_scale
