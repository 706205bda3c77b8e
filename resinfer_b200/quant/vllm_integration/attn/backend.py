"""vLLM attention backend: stock FlashInfer prefill and KV-cache writes, ResAttn decode.

Mirrors the reference's backend (ShawRong/ResInfer quant/vllm_integration/attn/backend.py:31-240):

* ``ResAttnFlashInferMetadataBuilder`` builds the stock metadata and refuses the batches the decode kernel does not
  take (cascade, DCP, more than one token per decode request, metadata that is not the TRTLLM form);
* ``ResAttnFlashInferImpl`` sends the prefill tokens of a step through the stock implementation and the decode
  tokens through ``ResAttnDecodeMixin`` -- BF16 output, or packed NVFP4 straight into the next projection's
  activation buffers when vLLM fused the output quantiser (head_dim 128);
* ``ResAttnFlashInferBackend`` names the two and narrows the supported configurations.

The KV cache is read where vLLM keeps it: every page holds K codes | K scales | V codes | V scales, and the four
strided views of it go to the kernel as they are (``ri_resattn_decode_strided``).

Written against the vLLM this image has (0.22: ``TRTLLMDecode``, ``nvfp4_kv_cache_split_views``); the names the
reference's vLLM (0.26) uses for the same things are tried first.  Two differences follow from 0.22: the stock
implementation wants the FP8 query it told the attention layer to produce, so with BF16 queries preserved for
decode this class quantises the prefill slice itself; and there is no CuTe-DSL warm-up registry, so the warm-up
provider is only kept (``warmup.py``).  Pages of 16, 32, 64 and 128 tokens are accepted (the reference: 128 only).
"""
from __future__ import annotations

import os
from dataclasses import replace

import torch

from vllm.model_executor.layers.quantization.utils.quant_utils import kNvfp4Dynamic
from vllm.utils.torch_utils import canonicalize_singleton_dim_strides
from vllm.v1.attention.backend import AttentionCGSupport
from vllm.v1.attention.backends.flashinfer import (
    FlashInferBackend,
    FlashInferImpl,
    FlashInferMetadata,
    FlashInferMetadataBuilder,
    TRTLLMPrefill,
)

try:                                                     # vLLM 0.26 names
    from vllm.v1.attention.backends.flashinfer import FlashInferDecodeKernel, FlashInferTrtllmAPIDecode as _TrtllmDecode
except ImportError:                                      # vLLM 0.22
    from vllm.v1.attention.backends.flashinfer import TRTLLMDecode as _TrtllmDecode
    FlashInferDecodeKernel = None

from ....nvfp4 import extension as _nvfp4_ext
from ....nvfp4.cute_attn.kv_layout import NvFp4PagedKVPool
from .decode import ResAttnDecodeMixin
from .warmup import _register_decode_warmup

_PAGE_SIZES = (16, 32, 64, 128)
_FP8 = torch.float8_e4m3fn


def _require_trtllm_decode(metadata):
    decode = metadata.decode
    ok = isinstance(decode, _TrtllmDecode)
    if ok and FlashInferDecodeKernel is not None:
        ok = decode.kernel is FlashInferDecodeKernel.TRTLLM_GEN
    if not ok:
        raise NotImplementedError("ResAttn requires stock FlashInfer TRTLLM_GEN decode metadata for NVFP4 KV")
    return decode


def _split_cache_views(kv_cache_hnd: torch.Tensor):
    """(k codes, k scales, v codes, v scales) of a cache permuted to [pages, 2, Hkv, page, 9 D / 16]."""
    try:
        from vllm.utils.torch_utils import nvfp4_kv_cache_split_views
        (kd, vd), (ks, vs) = nvfp4_kv_cache_split_views(kv_cache_hnd)
    except ImportError:
        from vllm.utils.torch_utils import nvfp4_split_data_scale
        kd, ks = nvfp4_split_data_scale(kv_cache_hnd[:, 0])
        vd, vs = nvfp4_split_data_scale(kv_cache_hnd[:, 1])
    return kd, ks, vd, vs


class ResAttnFlashInferMetadataBuilder(FlashInferMetadataBuilder):
    @classmethod
    def get_cudagraph_support(cls, vllm_config, kv_cache_spec):
        if os.environ.get("RESIDUE_ATTN_CUDAGRAPH", "0") == "1":
            return AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE
        return AttentionCGSupport.NEVER

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        if vllm_config.parallel_config.decode_context_parallel_size != 1:
            raise NotImplementedError("ResAttn decode does not support DCP")
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self._init_reorder_batch_threshold(1, supports_spec_as_decode=False)
        self._cg_capture_seq_len = (int(os.environ.get("RESIDUE_ATTN_CG_CAPTURE_LEN", "0"))
                                    or vllm_config.model_config.max_model_len)

    @staticmethod
    def _check(stock: FlashInferMetadata) -> FlashInferMetadata:
        """What ``build`` demands of the stock metadata (also used on metadata built elsewhere)."""
        if stock.use_cascade or not getattr(stock, "causal", True):
            raise NotImplementedError("ResAttn requires causal, non-cascade attention")
        if stock.num_prefill_tokens and not isinstance(stock.prefill, TRTLLMPrefill):
            raise NotImplementedError("This adapter requires stock TRTLLM prefill")
        n = stock.num_decodes
        if n:
            if n != stock.num_decode_tokens:
                raise NotImplementedError("ResAttn requires one token per decode")
            table = _require_trtllm_decode(stock).block_tables
            if (table.dtype != torch.int32 or table.ndim != 2 or table.shape[0] != n or table.shape[1] < 1
                    or table.stride(1) != 1 or table.stride(0) < table.shape[1]):
                raise ValueError("Expected int32 block table with unit column stride")
        return stock

    @staticmethod
    def _host_seq_lens(common_attn_metadata, n):
        """The decode requests' lengths as host integers when vLLM has them on the host already (no device
        synchronisation is ever made for them), else None.  Decode requests come first in the batch."""
        for name in ("seq_lens_cpu_upper_bound", "_seq_lens_cpu"):
            t = getattr(common_attn_metadata, name, None)
            if t is not None and t.shape[0] >= n:
                return [int(v) for v in t[:n].tolist()]
        return None

    def build(self, common_prefix_len, common_attn_metadata, fast_build=False) -> FlashInferMetadata:
        md = self._check(super().build(common_prefix_len, common_attn_metadata, fast_build))
        if md.num_decodes:                               # lets the split plan count the real tiles (plan.py)
            md.decode.seq_lens_host = self._host_seq_lens(common_attn_metadata, md.num_decodes)
        return md

    def build_for_cudagraph_capture(self, common_attn_metadata):
        md = self.build(0, common_attn_metadata)
        if md.num_decodes:                               # capture with the split plan of the longest sequence served
            decode = _require_trtllm_decode(md)
            decode.max_seq_len = max(decode.max_seq_len, self._cg_capture_seq_len)
            decode.seq_lens_host = None                  # the captured plan must not depend on this batch's lengths
        return md


class ResAttnFlashInferImpl(ResAttnDecodeMixin, FlashInferImpl):
    can_return_lse_for_decode = False

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        ok = self.num_kv_heads > 0 and self.num_heads % self.num_kv_heads == 0
        gqa = self.num_heads // self.num_kv_heads if ok else 0
        if not self.is_kvcache_nvfp4 or self.head_size not in (128, 256) or gqa not in (4, 6, 8):
            raise NotImplementedError("ResAttn candidate requires NVFP4, D128/D256, and GQA4/6/8")
        if (self.alibi_slopes is not None or self.window_left != -1 or self.logits_soft_cap not in (None, 0.0)
                or self.sinks is not None or self.kv_sharing_target_layer_name is not None):
            raise NotImplementedError("Unsupported ResAttn decode attention variant")
        # decode wants the BF16 query; set after super().__init__, which sets an instance value
        self.supports_quant_query_input = False
        self._decode_reduction_workspaces = {}
        self._residue_pool_key = None
        self._residue_pool = None
        _register_decode_warmup(self.num_heads, self.num_kv_heads, self.head_size)

    def fused_output_quant_supported(self, quant_key):
        return bool(self.is_kvcache_nvfp4 and self.head_size == 128 and quant_key == kNvfp4Dynamic)

    def _pool_for(self, kv_cache, layer):
        """The cache as four strided views; rebuilt only when the cache tensor or its scales change."""
        key = (kv_cache.data_ptr(), tuple(kv_cache.shape), kv_cache.stride(),
               float(layer._k_scale_float), float(layer._v_scale_float))
        if key != self._residue_pool_key:
            order = FlashInferBackend.get_kv_cache_stride_order()
            hnd = canonicalize_singleton_dim_strides(kv_cache.permute(*order))
            kd, ks, vd, vs = _split_cache_views(hnd)
            page = int(kd.shape[2])
            if (tuple(kd.shape[1:]) != (self.num_kv_heads, page, self.head_size // 2) or page not in _PAGE_SIZES
                    or tuple(kd.stride()[1:]) != (page * (self.head_size // 2), self.head_size // 2, 1)):
                raise ValueError("ResAttn requires the stock HND cache with pages of 16/32/64/128 tokens and a "
                                 f"matching head dimension, got shape {tuple(kd.shape)} strides {tuple(kd.stride())}")
            self._residue_pool = NvFp4PagedKVPool(
                num_kv_heads=self.num_kv_heads, head_dim=self.head_size, k_data=kd, v_data=vd, k_sf=ks, v_sf=vs,
                page_size=page, k_global_scale=key[-2], v_global_scale=key[-1])
            self._residue_pool_key = key
        return self._residue_pool

    def _stock_prefill_query(self, layer, q, md):
        """The stock implementation wants the query in the type its metadata names.  vLLM versions that let the
        implementation convert do so themselves; where the attention layer would have done it (and was told not
        to, for decode's sake) the prefill slice is converted here with the layer's static query scale."""
        want = getattr(md, "q_data_type", q.dtype)
        if want == q.dtype:
            return q
        if want != _FP8:
            raise ValueError(f"stock prefill wants {want} queries, got {q.dtype}")
        inv = 1.0 / float(layer._q_scale_float)
        fp8_max = torch.finfo(_FP8).max
        return (q.float() * inv).clamp_(-fp8_max, fp8_max).to(_FP8)

    def _tokens_heads_dim(self, t):
        return t if t.dim() == 3 else t.view(-1, self.num_heads, self.head_size)

    def _decode_query(self, query, md):
        """The decode tokens' queries as one dense [n, Hq, D] block (vLLM hands a strided slice of the fused QKV
        output; the kernel reads whole rows with the copy engine)."""
        q = self._tokens_heads_dim(query)[:md.num_decode_tokens]
        return q if q.is_contiguous() else q.contiguous()

    def _pack_nvfp4(self, bf16_output, n, output, output_scale, output_block_scale):
        """Quantise [n, Hq, D] BF16 into the packed activation buffers (codes + 128x4 block scales)."""
        hidden = self.num_heads * self.head_size
        _nvfp4_ext.ensure_loaded()
        torch.ops.nvfp4.scaled_fp4_quant_mext_r1(
            output[:n].reshape(n, hidden // 2).view(torch.uint8), bf16_output[:n].reshape(n, hidden),
            output_block_scale.view(torch.uint8), output_scale, 0, 5, True)      # layout 5: base codes only

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                output_block_scale=None):
        if output_scale is None and output_block_scale is None:
            scales = None
        elif output_scale is not None and output_block_scale is not None:
            scales = (output_scale, output_block_scale)
        else:
            raise ValueError("NVFP4 attention output requires data and block scales")
        if attn_metadata is None:                        # profiling run
            return output.fill_(0)
        if query.dtype != torch.bfloat16:
            raise ValueError("ResAttn needs original BF16 Q, not FP8 Q")
        if output.dtype != (torch.uint8 if scales is not None else torch.bfloat16):
            raise ValueError("ResAttn output dtype does not match fusion mode")
        md = attn_metadata
        if md.num_prefill_tokens:
            # the step's K/V are in the cache already; decodes come first in the batch, prefills after
            bf16_output = output if scales is None else torch.empty_like(query)
            n, end = md.num_decode_tokens, md.num_actual_tokens
            prefill_md, q_pre, k_pre, v_pre, prefill_output = md, query, key, value, bf16_output
            if md.num_decodes:
                prefill_md = replace(md, num_actual_tokens=md.num_prefill_tokens, num_decodes=0, num_decode_tokens=0,
                                     decode=None, slot_mapping=md.slot_mapping[n:end])
                q_pre, k_pre, v_pre = query[n:end], key[n:end], value[n:end]
                prefill_output = bf16_output[n:end]
            FlashInferImpl.forward(self, layer, self._stock_prefill_query(layer, q_pre, prefill_md), k_pre, v_pre,
                                   kv_cache, prefill_md, prefill_output)
            if md.num_decodes:
                _require_trtllm_decode(md)
                self._decode_forward(self._decode_query(query, md), self._pool_for(kv_cache, layer), md,
                                     self._tokens_heads_dim(bf16_output))
            if scales is not None:
                self._pack_nvfp4(bf16_output, md.num_actual_tokens, output, *scales)
            return output
        if md.num_decodes:
            _require_trtllm_decode(md)
            pool = self._pool_for(kv_cache, layer)
            q = self._decode_query(query, md)
            if scales is not None:
                self._decode_forward_nvfp4(q, pool, md, output, *scales)
            else:
                self._decode_forward(q, pool, md, self._tokens_heads_dim(output))
        return output


class ResAttnFlashInferBackend(FlashInferBackend):
    """Stock prefill and cache contract with ResAttn decode, mixed batches included."""
    supported_dtypes = [torch.bfloat16]
    supported_kv_cache_dtypes = ["nvfp4"]

    @staticmethod
    def get_name():
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return ResAttnFlashInferImpl

    @staticmethod
    def get_builder_cls():
        return ResAttnFlashInferMetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes():
        return list(_PAGE_SIZES)

    @classmethod
    def get_supported_head_sizes(cls):
        return [128, 256]

    @classmethod
    def supports_sink(cls):
        return False
