"""The decode half of the attention adapter (``ResAttnDecodeMixin``: the two methods the reference's vLLM
attention implementation calls, quant/vllm_integration/attn/decode.py:55-165) driven with plain objects in
place of vLLM's metadata: BF16 output against the oracle, packed NVFP4 output against the oracle's
quantisation of the BF16 path's unrounded result, and the per-layer workspace cache."""
import types

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _layer(hq, hkv, d):
    from resinfer_b200.quant.vllm_integration.attn import ResAttnDecodeMixin

    class Impl(ResAttnDecodeMixin):
        def __init__(self):
            self.num_heads, self.num_kv_heads, self.head_size = hq, hkv, d
            self.scale = d ** -0.5
            self._decode_reduction_workspaces = {}
    return Impl()


def test_decode_mixin_bf16_and_nvfp4(cuda_device, device_rcp):
    from resinfer_b200 import ops
    from resinfer_b200.nvfp4.cute_attn.host import allocate_nvfp4_attention_output
    from resinfer_b200.nvfp4.cute_attn.kv_layout import NvFp4PagedKVPool
    d, page, hkv, g = 128, 16, 2, 8
    lens = [5000, 300, 1700, 64, 2049]
    n_dec = 4                                                  # the step carries one more (prefill) token row
    kv = O.make_paged_kv(lens[:n_dec], hkv, d, page, seed=31)
    hq = hkv * g
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)   # noqa: E731
    q_np = O.bf16_round(np.random.default_rng(8).standard_normal((n_dec + 1, hq, d)).astype(np.float32))
    pool = NvFp4PagedKVPool(hkv, d, t(kv["k_data"]), t(kv["v_data"]), t(kv["k_sf"]), t(kv["v_sf"]), page_size=page,
                            k_global_scale=kv["k_global_scale"], v_global_scale=kv["v_global_scale"])
    md = types.SimpleNamespace(num_decode_tokens=n_dec, decode=types.SimpleNamespace(
        block_tables=t(np.maximum(kv["block_tables"], 0)), seq_lens=t(kv["seq_lens"]), max_seq_len=max(lens[:n_dec])))
    layer = _layer(hq, hkv, d)
    q_all = t(q_np).to(torch.bfloat16)
    out3 = torch.zeros(n_dec + 1, hq, d, dtype=torch.bfloat16, device=cuda_device)
    layer._decode_forward(q_all, pool, md, out3)
    torch.cuda.synchronize()
    ops.check_status(cuda_device)
    ref = O.resattn_decode_reference(q_np[:n_dec], kv, d ** -0.5, rcp=O.RecordingRcp(device_rcp))
    assert rel_fro(out3[:n_dec].float().cpu().numpy(), ref) < 3e-3
    assert not out3[n_dec].any()                                # rows past the decode tokens stay untouched
    # the workspace of the plan is cached on the layer: a second call allocates nothing new
    cached = dict(layer._decode_reduction_workspaces)
    layer._decode_forward(q_all, pool, md, out3)
    assert layer._decode_reduction_workspaces.keys() == cached.keys()
    assert all(layer._decode_reduction_workspaces[k] is v for k, v in cached.items())
    # ---- packed NVFP4 output into caller-owned activation buffers
    packed, block_scale = allocate_nvfp4_attention_output(n_dec + 1, hq, d, cuda_device)
    gs = 6.0 * 448.0 / float(out3[:n_dec].float().abs().max())
    gsi = torch.tensor([gs], dtype=torch.float32, device=cuda_device)
    layer._decode_forward_nvfp4(q_all, pool, md, packed, gsi, block_scale)
    torch.cuda.synchronize()
    ops.check_status(cuda_device)
    sf = block_scale.view(torch.uint8).reshape(-1).cpu().numpy()
    deq = O.nvfp4_dequant(packed[:n_dec].cpu().numpy(), O.unswizzle_scales(sf, n_dec, hq * d // 16), 1.0 / gs)
    assert rel_fro(deq, ref.reshape(n_dec, -1)) < 0.12          # FP4 error of the output quantisation
    with pytest.raises(ValueError, match="unsupported persistent reduction"):
        layer._get_decode_reduction_workspace(None, 2, 1, cuda_device, reduction="cga_sharded")
