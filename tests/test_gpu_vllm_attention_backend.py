"""The vLLM attention backend's decode on the GPU, over a cache laid out the way vLLM keeps it: every page holds
K codes | K scales | V codes | V scales, and ``ResAttnFlashInferImpl`` hands the kernel four strided views of it
(``ri_resattn_decode_strided``).  Checked against the oracle, and bit for bit against the same decode over a
densely repacked copy of the cache -- the strides must change nothing but addresses.  Pages of 128 tokens go
through the tiled copy engine (3-D tensor map), smaller ones through ``cp.async``.  The stock prefill is replaced by
a recorder (it needs a vLLM engine around it); ``FlashInferImpl.__init__`` by its attribute assignments (its
platform queries want a vLLM configuration)."""
import types

import numpy as np
import pytest
import torch

import oracle as O

pytest.importorskip("vllm")
pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _stock_init(self, num_heads, head_size, scale, num_kv_heads, alibi_slopes=None, sliding_window=None,
                kv_cache_dtype="nvfp4", logits_soft_cap=None, attn_type=None, kv_sharing_target_layer_name=None,
                sinks=None):
    self.num_heads, self.head_size, self.scale, self.num_kv_heads = num_heads, head_size, float(scale), num_kv_heads
    self.alibi_slopes, self.window_left = alibi_slopes, -1
    self.kv_cache_dtype, self.is_kvcache_nvfp4 = kv_cache_dtype, kv_cache_dtype == "nvfp4"
    self.logits_soft_cap, self.kv_sharing_target_layer_name, self.sinks = logits_soft_cap, kv_sharing_target_layer_name, sinks


@pytest.fixture()
def impl_cls(monkeypatch):
    from vllm.v1.attention.backends.flashinfer import FlashInferBackend, FlashInferImpl
    from resinfer_b200.quant.vllm_integration.attn import backend
    monkeypatch.setattr(FlashInferImpl, "__init__", _stock_init)
    monkeypatch.setattr(FlashInferBackend, "get_kv_cache_stride_order", staticmethod(lambda *a, **k: (0, 1, 3, 2, 4)))
    return backend.ResAttnFlashInferImpl


def _vllm_cache(kv, dev, extra_pages=3):
    """The oracle's pool written into vLLM's cache: memory [pages, 2, Hkv * page * d/2 codes | Hkv * page * d/16
    scales], handed out as the logical [pages, 2, page, Hkv, 9 d / 16] view of it.  Unused pages hold noise."""
    pages, hkv, page, half = kv["k_data"].shape
    d = 2 * half
    full = half + d // 16
    total = pages + extra_pages
    mem = torch.randint(0, 256, (total, 2, hkv * page * full), dtype=torch.uint8,
                        generator=torch.Generator().manual_seed(5))
    for side, (codes, sf) in enumerate(((kv["k_data"], kv["k_sf"]), (kv["v_data"], kv["v_sf"]))):
        mem[:pages, side, :hkv * page * half] = torch.from_numpy(np.ascontiguousarray(codes)).reshape(pages, -1)
        mem[:pages, side, hkv * page * half:] = torch.from_numpy(np.ascontiguousarray(sf)).reshape(pages, -1)
    mem = mem.to(dev)
    return mem.view(total, 2, hkv, page, full).permute(0, 1, 3, 2, 4), mem


def _metadata(kv, n_dec, dev, n_prefill=0):
    from vllm.v1.attention.backends import flashinfer as fi
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)   # noqa: E731
    dec = fi.TRTLLMDecode(block_tables=t(np.maximum(kv["block_tables"], 0))[:n_dec], seq_lens=t(kv["seq_lens"])[:n_dec],
                          max_seq_len=int(kv["seq_lens"][:n_dec].max()))
    pre = None
    if n_prefill:
        z = torch.zeros(2, dtype=torch.int32, device=dev)
        pre = fi.TRTLLMPrefill(block_tables=dec.block_tables[:1], seq_lens=z[:1], cum_seq_lens_q=z, cum_seq_lens_kv=z,
                               max_q_len=n_prefill, max_seq_len=n_prefill)
    total = n_dec + n_prefill
    return fi.FlashInferMetadata(
        num_actual_tokens=total, slot_mapping=torch.arange(total, device=dev), q_data_type=torch.float8_e4m3fn,
        num_decodes=n_dec, num_decode_tokens=n_dec, num_prefills=1 if n_prefill else 0, num_prefill_tokens=n_prefill,
        prefill=pre, decode=dec, use_cascade=False, cascade_wrapper=None)


def _dense_pool(kv, dev, page):
    from resinfer_b200.nvfp4.cute_attn.kv_layout import NvFp4PagedKVPool
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)   # noqa: E731
    hkv, d = kv["k_data"].shape[1], 2 * kv["k_data"].shape[3]
    return NvFp4PagedKVPool(hkv, d, t(kv["k_data"]), t(kv["v_data"]), t(kv["k_sf"]), t(kv["v_sf"]), page_size=page,
                            k_global_scale=kv["k_global_scale"], v_global_scale=kv["v_global_scale"])


@pytest.mark.parametrize("d,page,hkv,g,lens", [
    (128, 128, 2, 8, [5000, 300, 1700, 129]),        # tiled copies with a page stride
    (128, 16, 2, 4, [700, 33, 1]),                   # cp.async path, a tile spans eight pages
    (256, 128, 1, 8, [2049, 640]),
    (128, 64, 3, 6, [1000, 64, 65, 4097, 12]),
    (256, 32, 2, 4, [513, 96]),
])
def test_decode_reads_the_vllm_cache_in_place(cuda_device, device_rcp, impl_cls, d, page, hkv, g, lens):
    from resinfer_b200 import ops
    dev = cuda_device
    kv = O.make_paged_kv(lens, hkv, d, page, seed=d + page)
    hq, n = hkv * g, len(lens)
    cache, _ = _vllm_cache(kv, dev)
    layer = types.SimpleNamespace(_k_scale_float=kv["k_global_scale"], _v_scale_float=kv["v_global_scale"], _q_scale_float=1.0)
    impl = impl_cls(hq, d, d ** -0.5, hkv)
    md = _metadata(kv, n, dev)
    q_np = O.bf16_round(np.random.default_rng(3).standard_normal((n + 2, hq, d)).astype(np.float32))
    q = torch.from_numpy(q_np).to(dev).to(torch.bfloat16)                 # two padding rows, as under a CUDA graph
    out = torch.zeros(n + 2, hq, d, dtype=torch.bfloat16, device=dev)
    assert impl.forward(layer, q, None, None, cache, md, out) is out
    torch.cuda.synchronize()
    ops.check_status(dev)
    ref = O.resattn_decode_reference(q_np[:n], kv, d ** -0.5, rcp=O.RecordingRcp(device_rcp))
    assert rel_fro(out[:n].float().cpu().numpy(), ref) < 3e-3
    assert not out[n:].any()
    # the same decode over a dense copy of the pool: identical bits
    dense = torch.zeros_like(out)
    impl._decode_forward(q[:n].contiguous(), _dense_pool(kv, dev, page), md, dense)
    torch.cuda.synchronize()
    assert torch.equal(out, dense)
    # a query that is a strided slice of a fused QKV buffer gives the same result
    qkv = torch.zeros(n + 2, 3, hq * d, dtype=torch.bfloat16, device=dev)
    qkv[:, 0] = q.view(n + 2, -1)
    out2 = torch.zeros_like(out)
    impl.forward(layer, qkv[:, 0].view(-1, hq, d), None, None, cache, md, out2.view(n + 2, hq * d))
    torch.cuda.synchronize()
    assert torch.equal(out2, out)


def test_strided_entry_rejects_bad_strides(cuda_device):
    from resinfer_b200 import _cabi, ops
    lib = _cabi.load()
    dev = cuda_device
    z = torch.zeros(4096, dtype=torch.uint8, device=dev)
    q = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device=dev)
    bt = torch.zeros(1, 1, dtype=torch.int32, device=dev)
    sl = torch.ones(1, dtype=torch.int32, device=dev)
    out = torch.zeros_like(q)

    def call(code_stride, sf_stride):
        return lib.ri_resattn_decode_strided(
            q.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, code_stride, sf_stride, bt.data_ptr(), 1,
            sl.data_ptr(), 1, 8, 1, 128, 16, 0, 1.0, 1.0, out.data_ptr(), _cabi.DTYPE_BF16, None, 0, None, 0, None, None, 0,
            1, _cabi.ATTN_REDUCER_TICKET, None, 0, 1, ops.status_word(dev).data_ptr(), _cabi.current_stream(dev))
    assert call(16 * 64 - 16, 0) != 0 and b"page strides" in lib.ri_last_error()       # smaller than a page
    assert call(16 * 64 + 8, 0) != 0                                                   # not a multiple of 16
    assert call(0, 16 * 8 + 4) != 0
    assert call(0, 0) == 0 and call(2048, 256) == 0
    torch.cuda.synchronize()
    assert lib.ri_resattn_prepare(64) != 0 and lib.ri_resattn_prepare(128) == 0 and lib.ri_resattn_prepare(256) == 0


def test_mixed_step_and_fused_nvfp4_output(cuda_device, device_rcp, impl_cls, monkeypatch):
    from vllm.v1.attention.backends.flashinfer import FlashInferImpl
    from resinfer_b200 import ops
    from resinfer_b200.nvfp4.cute_attn.host import allocate_nvfp4_attention_output
    dev = cuda_device
    d, page, hkv, g = 128, 128, 2, 8
    lens = [900, 4000, 130]
    n_dec, n_pre = len(lens), 6
    total = n_dec + n_pre
    hq = hkv * g
    kv = O.make_paged_kv(lens, hkv, d, page, seed=77)
    cache, _ = _vllm_cache(kv, dev)
    layer = types.SimpleNamespace(_k_scale_float=kv["k_global_scale"], _v_scale_float=kv["v_global_scale"], _q_scale_float=0.25)
    impl = impl_cls(hq, d, d ** -0.5, hkv)
    prefill_value = (torch.randn(n_pre, hq, d, device=dev) * 0.5).to(torch.bfloat16)
    seen = {}

    def stock_forward(self, layer_, query, key, value, kv_cache, md, output, output_scale=None, output_block_scale=None):
        seen.update(q_dtype=query.dtype, tokens=md.num_actual_tokens, decodes=md.num_decodes, slots=md.slot_mapping.tolist())
        output.copy_(prefill_value)
        return output
    monkeypatch.setattr(FlashInferImpl, "forward", stock_forward)
    md = _metadata(kv, n_dec, dev, n_prefill=n_pre)
    q_np = O.bf16_round(np.random.default_rng(4).standard_normal((total, hq, d)).astype(np.float32))
    q = torch.from_numpy(q_np).to(dev).to(torch.bfloat16)
    kx = torch.zeros(total, hkv, d, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(total, hq, d, dtype=torch.bfloat16, device=dev)
    impl.forward(layer, q, kx, kx, cache, md, out)
    torch.cuda.synchronize()
    ops.check_status(dev)
    assert seen == dict(q_dtype=torch.float8_e4m3fn, tokens=n_pre, decodes=0, slots=list(range(n_dec, total)))
    ref = O.resattn_decode_reference(q_np[:n_dec], kv, d ** -0.5, rcp=O.RecordingRcp(device_rcp))
    assert rel_fro(out[:n_dec].float().cpu().numpy(), ref) < 3e-3
    assert torch.equal(out[n_dec:], prefill_value)

    # fused output quantiser, mixed step: one quantisation over decode and prefill rows together
    packed, block_scale = allocate_nvfp4_attention_output(total, hq, d, dev)
    gs = 6.0 * 448.0 / float(out.float().abs().max())
    gsi = torch.tensor([gs], dtype=torch.float32, device=dev)
    impl.forward(layer, q, kx, kx, cache, md, packed, output_scale=gsi, output_block_scale=block_scale)
    torch.cuda.synchronize()
    ops.check_status(dev)
    sf = block_scale.view(torch.uint8).reshape(-1).cpu().numpy()
    codes_want, sf_want = O.nvfp4_quant_plain(out.float().cpu().numpy().reshape(total, -1), gs, rcp=O.RecordingRcp(device_rcp))
    assert np.array_equal(packed.cpu().numpy(), codes_want)
    assert np.array_equal(O.unswizzle_scales(sf, total, hq * d // 16), O.unswizzle_scales(sf_want, total, hq * d // 16))

    # fused output quantiser, decode only: the kernel writes the packed activations itself
    md_dec = _metadata(kv, n_dec, dev)
    packed2, block_scale2 = allocate_nvfp4_attention_output(n_dec, hq, d, dev)
    impl.forward(layer, q[:n_dec], kx[:n_dec], kx[:n_dec], cache, md_dec, packed2, output_scale=gsi, output_block_scale=block_scale2)
    dense_packed, dense_scale = allocate_nvfp4_attention_output(n_dec, hq, d, dev)
    impl._decode_forward_nvfp4(q[:n_dec].contiguous(), _dense_pool(kv, dev, page), md_dec, dense_packed, gsi, dense_scale)
    torch.cuda.synchronize()
    ops.check_status(dev)
    assert torch.equal(packed2, dense_packed) and torch.equal(block_scale2.view(torch.uint8), dense_scale.view(torch.uint8))
    deq = O.nvfp4_dequant(packed2.cpu().numpy(), O.unswizzle_scales(block_scale2.view(torch.uint8).reshape(-1).cpu().numpy(),
                                                                    n_dec, hq * d // 16), 1.0 / gs)
    assert rel_fro(deq, ref.reshape(n_dec, -1)) < 0.12


def test_warmup_units_run(cuda_device):
    from resinfer_b200.quant.vllm_integration.attn import warmup
    prov = warmup._DecodeWarmupProvider()
    prov.add_geometry(32, 8, 128, False)
    prov.add_geometry(32, 8, 256, False)
    with torch.cuda.device(cuda_device):
        assert prov.warm_now() == 2
