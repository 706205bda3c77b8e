"""ResAttn decode launches for an attention implementation class.

``ResAttnDecodeMixin`` carries the two methods the reference's vLLM attention implementation calls for
the decode tokens of a step (ShawRong/ResInfer quant/vllm_integration/attn/decode.py:55-165):
``_decode_forward`` (BF16 output) and ``_decode_forward_nvfp4`` (packed NVFP4 output straight into the
activation buffers of the following projection), plus the per-layer cache of split-KV reduction
workspaces (:23-53).  The host class supplies ``num_heads``, ``num_kv_heads``, ``head_size``, ``scale``
and a dict ``_decode_reduction_workspaces``; the metadata object supplies ``num_decode_tokens`` and
``decode.block_tables / seq_lens / max_seq_len`` (and, optionally, ``decode.seq_lens_host``: the lengths as host
integers for the split plan, this library's addition); ``pool`` is an ``NvFp4PagedKVPool``.

Nothing here imports vLLM, so the mixin can be exercised with plain objects; the vLLM-facing classes
(metadata builder, prefill through the stock implementation) are in ``backend.py``.
"""
from __future__ import annotations

import torch

from ....nvfp4.cute_attn import host as _host

_PERSISTENT_REDUCERS = ("kernel", "gmem_fused")


def _decode_slice(q_all: torch.Tensor, n: int) -> torch.Tensor:
    return q_all if q_all.shape[0] == n else q_all[:n]


class ResAttnDecodeMixin:
    num_heads: int
    num_kv_heads: int
    head_size: int
    scale: float
    _decode_reduction_workspaces: dict

    def _get_decode_reduction_workspace(self, host, splits: int, batch: int, device, reduction: str = "kernel"):
        """Partial (o, l, m) buffers for ``splits`` KV splits of ``batch`` sequences, allocated once per
        (reducer, splits, batch, padded head count, device) and kept on the layer."""
        if reduction not in _PERSISTENT_REDUCERS:
            raise ValueError(f"unsupported persistent reduction: {reduction}")
        # the kernel's Q tile pads every GQA group (8 rows for GQA4, 16 otherwise): size for the padded heads
        heads = self.num_kv_heads * host._residue_padded_group_size(self.num_heads, self.num_kv_heads)
        key = (reduction, splits, batch, heads, str(device))
        ws = self._decode_reduction_workspaces.get(key)
        if ws is None:
            ws = host.allocate_qmul4_reduction_workspace(splits, batch, heads, self.head_size, device)
            self._decode_reduction_workspaces[key] = ws
        return ws

    def _decode_forward(self, q_all, pool, md, out3) -> None:
        """Decode tokens -> ``out3[:n]`` (BF16 [n, Hq, D]); the KV cache already holds this step's tokens."""
        n = md.num_decode_tokens
        dec = md.decode
        q = _decode_slice(q_all, n)
        _host.check_shape_supported(self.num_heads, self.num_kv_heads, self.head_size)
        plan, ws = None, None
        if dec.max_seq_len:                                   # unknown length: the host entry plans by itself
            plan = _host.plan_qmul4_decode(
                n, self.num_kv_heads, dec.max_seq_len, q.device, head_dim=self.head_size,
                grouped_head_tile=_host._residue_padded_group_size(self.num_heads, self.num_kv_heads),
                seq_lens=getattr(dec, "seq_lens_host", None))
            if plan[1] == "kernel":
                ws = self._get_decode_reduction_workspace(_host, plan[0], n, q.device)
        _host.run_paged_fp4_decode_qmul4_tmem(
            q, pool, pool.v_data, pool.v_sf, dec.block_tables, dec.seq_lens, self.scale * pool.k_global_scale,
            out=out3[:n], max_seq_len=dec.max_seq_len, k_sf_mode="linear", value_scale=pool.v_global_scale,
            reduction_workspace=ws, plan=plan)

    def _decode_forward_nvfp4(self, q_all, pool, md, output, output_scale, output_block_scale) -> None:
        """Decode tokens -> packed NVFP4 codes in ``output[:n]`` and their 128x4 block scales, the activation
        format of the projection that follows (head_dim 128)."""
        n = md.num_decode_tokens
        dec = md.decode
        q = _decode_slice(q_all, n)
        _host.check_shape_supported(self.num_heads, self.num_kv_heads, self.head_size)
        plan = _host.plan_qmul4_decode_nvfp4(n, self.num_heads, self.num_kv_heads, dec.max_seq_len, q.device,
                                             seq_lens=getattr(dec, "seq_lens_host", None))
        ws = None
        if plan[1] in _PERSISTENT_REDUCERS:
            ws = self._get_decode_reduction_workspace(_host, plan[0], n, q.device, reduction=plan[1])
        rows = (n + 127) // 128 * 128
        _host.run_paged_fp4_decode_qmul4_tmem_nvfp4(
            q, pool, pool.v_data, pool.v_sf, dec.block_tables, dec.seq_lens, self.scale * pool.k_global_scale,
            output_scale, out=output[:n].view(n, self.num_heads * self.head_size // 2),
            output_block_scale=output_block_scale[:rows], max_seq_len=dec.max_seq_len, k_sf_mode="linear",
            value_scale=pool.v_global_scale, reduction_workspace=ws, plan=plan)
