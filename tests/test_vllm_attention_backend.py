"""The vLLM attention backend (``resinfer_b200.quant.vllm_integration.attn``) on CPU: registration, what the
metadata builder refuses, the constructor's refusals, the views cut out of vLLM's interleaved NVFP4 cache, and how
``forward`` divides a step between the stock prefill and the decode mixin (both replaced by recorders here; the
kernels run in tests/test_gpu_vllm_attention_backend.py).  Follows the reference's adapter
(ShawRong/ResInfer quant/vllm_integration/attn/backend.py, register.py, warmup.py)."""
import types

import pytest
import torch

pytest.importorskip("vllm")

from resinfer_b200.quant.vllm_integration.attn import register  # noqa: E402


# ------------------------------------------------------------------------------------------------ registration
class _FakeEnumMember:
    def __init__(self):
        self.path = None

    def is_overridden(self):
        return self.path is not None

    def get_path(self):
        return self.path


def _fake_registry(custom_path=None):
    custom = _FakeEnumMember()
    custom.path = custom_path
    enum = types.SimpleNamespace(__members__={"CUSTOM": custom}, CUSTOM=custom)
    reg = types.SimpleNamespace(AttentionBackendEnum=enum)

    def register_backend(backend, class_path=None):
        backend.path = class_path
    reg.register_backend = register_backend
    return reg


def test_install_is_gated_by_the_environment(monkeypatch):
    monkeypatch.delenv("RESIDUE_ATTN", raising=False)
    reg = _fake_registry()
    assert register.install(registry=reg) is False and reg.AttentionBackendEnum.CUSTOM.path is None
    monkeypatch.setenv("RESIDUE_ATTN", "1")
    assert register.install(registry=reg) is True
    assert reg.AttentionBackendEnum.CUSTOM.path == register._BACKEND_CLASS_PATH
    assert register.install(registry=reg) is True                      # second call: already installed


def test_install_refuses_a_foreign_custom_backend_and_odd_registries():
    reg = _fake_registry("somebody.else.Backend")
    assert register.install(force=True, registry=reg) is False
    assert reg.AttentionBackendEnum.CUSTOM.path == "somebody.else.Backend"
    assert register.install(force=True, registry=types.SimpleNamespace()) is False
    no_custom = _fake_registry()
    no_custom.AttentionBackendEnum.__members__ = {}
    assert register.install(force=True, registry=no_custom) is False
    changed = _fake_registry()
    changed.register_backend = lambda backend, path=None: None         # another signature
    assert register.install(force=True, registry=changed) is False


def test_install_into_the_real_registry_resolves_to_the_backend_class():
    import vllm.v1.attention.backends.registry as reg
    assert not reg.AttentionBackendEnum.CUSTOM.is_overridden()
    try:
        assert register.install(force=True) is True
        cls = reg.AttentionBackendEnum.CUSTOM.get_class()
        from resinfer_b200.quant.vllm_integration.attn.backend import ResAttnFlashInferBackend
        assert cls is ResAttnFlashInferBackend and cls.get_name() == "CUSTOM"
    finally:
        reg._ATTN_OVERRIDES.pop(reg.AttentionBackendEnum.CUSTOM, None)
        if hasattr(reg, register._INSTALLED_ATTR):
            delattr(reg, register._INSTALLED_ATTR)


def test_plugin_registers_the_backend(monkeypatch):
    import vllm.v1.attention.backends.registry as reg
    from resinfer_b200.runtime.vllm_plugin import residue_vllm_plugin as plugin
    for k in ("RESIDUE_NVFP4", "RESIDUE_MXFP4"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("RESIDUE_ATTN", "1")
    import resinfer_b200.nvfp4.extension as ext
    monkeypatch.setattr(ext, "ensure_loaded", lambda required=True: True)     # no GPU library calls here
    try:
        plugin.initialize()
        assert reg.AttentionBackendEnum.CUSTOM.get_path() == register._BACKEND_CLASS_PATH
    finally:
        reg._ATTN_OVERRIDES.pop(reg.AttentionBackendEnum.CUSTOM, None)
        if hasattr(reg, register._INSTALLED_ATTR):
            delattr(reg, register._INSTALLED_ATTR)


# ------------------------------------------------------------------------------------------- backend declarations
def test_backend_declarations():
    from vllm.v1.attention.backend import AttentionBackend
    from resinfer_b200.quant.vllm_integration.attn.backend import (
        ResAttnFlashInferBackend, ResAttnFlashInferImpl, ResAttnFlashInferMetadataBuilder)
    b = ResAttnFlashInferBackend
    assert issubclass(b, AttentionBackend)
    assert b.get_impl_cls() is ResAttnFlashInferImpl and b.get_builder_cls() is ResAttnFlashInferMetadataBuilder
    assert b.supported_dtypes == [torch.bfloat16] and b.supported_kv_cache_dtypes == ["nvfp4"]
    assert b.get_supported_head_sizes() == [128, 256] and b.supports_sink() is False
    assert 128 in b.get_supported_kernel_block_sizes()
    # the cache shape is the stock one: data and block scales packed in the last dimension
    assert b.get_kv_cache_shape(10, 128, 8, 128, "nvfp4") == (10, 2, 128, 8, 72)
    assert ResAttnFlashInferImpl.can_return_lse_for_decode is False


def test_cudagraph_support_follows_the_environment(monkeypatch):
    from vllm.v1.attention.backend import AttentionCGSupport
    from resinfer_b200.quant.vllm_integration.attn.backend import ResAttnFlashInferMetadataBuilder as Bld
    monkeypatch.delenv("RESIDUE_ATTN_CUDAGRAPH", raising=False)
    assert Bld.get_cudagraph_support(None, None) is AttentionCGSupport.NEVER
    monkeypatch.setenv("RESIDUE_ATTN_CUDAGRAPH", "1")
    assert Bld.get_cudagraph_support(None, None) is AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE


# -------------------------------------------------------------------------------------------------- the builder
def _metadata(num_decodes=3, num_prefill_tokens=0, decode="trtllm", tokens_per_decode=1, table=None, prefill="trtllm",
              cascade=False):
    from vllm.v1.attention.backends import flashinfer as fi
    n_dec_tok = num_decodes * tokens_per_decode
    if table is None:
        table = torch.zeros(max(num_decodes, 1), 4, dtype=torch.int32)[:num_decodes]
    dec = None
    if num_decodes:
        if decode == "trtllm":
            dec = fi.TRTLLMDecode(block_tables=table, seq_lens=torch.ones(num_decodes, dtype=torch.int32), max_seq_len=77)
        else:
            dec = fi.FIDecode(wrapper=None)
    pre = None
    if num_prefill_tokens:
        if prefill == "trtllm":
            z = torch.zeros(2, dtype=torch.int32)
            pre = fi.TRTLLMPrefill(block_tables=torch.zeros(1, 4, dtype=torch.int32), seq_lens=z[:1], cum_seq_lens_q=z,
                                   cum_seq_lens_kv=z, max_q_len=num_prefill_tokens, max_seq_len=num_prefill_tokens)
        else:
            pre = fi.FIPrefill(wrapper=None)
    total = n_dec_tok + num_prefill_tokens
    return fi.FlashInferMetadata(
        num_actual_tokens=total, slot_mapping=torch.arange(total), q_data_type=torch.float8_e4m3fn,
        num_decodes=num_decodes, num_decode_tokens=n_dec_tok, num_prefills=1 if num_prefill_tokens else 0,
        num_prefill_tokens=num_prefill_tokens, prefill=pre, decode=dec, use_cascade=cascade, cascade_wrapper=None)


def test_builder_accepts_the_stock_trtllm_metadata_and_refuses_the_rest():
    from resinfer_b200.quant.vllm_integration.attn.backend import ResAttnFlashInferMetadataBuilder as Bld
    md = _metadata()
    assert Bld._check(md) is md
    assert Bld._check(_metadata(num_decodes=2, num_prefill_tokens=9)).num_prefill_tokens == 9
    assert Bld._check(_metadata(num_decodes=0, num_prefill_tokens=5)).decode is None
    with pytest.raises(NotImplementedError, match="cascade"):
        Bld._check(_metadata(cascade=True))
    with pytest.raises(NotImplementedError, match="one token per decode"):
        Bld._check(_metadata(tokens_per_decode=2))
    with pytest.raises(NotImplementedError, match="TRTLLM_GEN decode"):
        Bld._check(_metadata(decode="native"))
    with pytest.raises(NotImplementedError, match="TRTLLM prefill"):
        Bld._check(_metadata(num_prefill_tokens=4, prefill="native"))
    with pytest.raises(ValueError, match="int32 block table"):
        Bld._check(_metadata(table=torch.zeros(3, 4, dtype=torch.int64)))
    with pytest.raises(ValueError, match="int32 block table"):
        Bld._check(_metadata(table=torch.zeros(3, 8, dtype=torch.int32)[:, ::2]))     # column stride 2
    with pytest.raises(ValueError, match="int32 block table"):
        Bld._check(_metadata(table=torch.zeros(2, 4, dtype=torch.int32)))             # rows != decodes


def test_builder_refuses_decode_context_parallel_and_lengthens_the_capture(monkeypatch):
    from vllm.v1.attention.backends.flashinfer import FlashInferMetadataBuilder
    from resinfer_b200.quant.vllm_integration.attn.backend import ResAttnFlashInferMetadataBuilder as Bld
    cfg = types.SimpleNamespace(parallel_config=types.SimpleNamespace(decode_context_parallel_size=2),
                                model_config=types.SimpleNamespace(max_model_len=4096), speculative_config=None)
    with pytest.raises(NotImplementedError, match="DCP"):
        Bld(None, [], cfg, "cpu")
    cfg.parallel_config.decode_context_parallel_size = 1

    def stock_init(self, kv_cache_spec, layer_names, vllm_config, device):
        self.vllm_config = vllm_config
    monkeypatch.setattr(FlashInferMetadataBuilder, "__init__", stock_init)
    monkeypatch.setattr(FlashInferMetadataBuilder, "build", lambda self, prefix, common, fast_build=False: common)
    monkeypatch.delenv("RESIDUE_ATTN_CG_CAPTURE_LEN", raising=False)
    b = Bld(None, [], cfg, "cpu")
    assert b.reorder_batch_threshold == 1 and b._cg_capture_seq_len == 4096
    md = b.build_for_cudagraph_capture(_metadata())                    # the fake stock build hands the metadata through
    assert md.decode.max_seq_len == 4096 and md.decode.seq_lens_host is None
    # host lengths, when vLLM has them, travel with the decode metadata for the split plan (never under capture)
    common = _metadata(num_decodes=3, num_prefill_tokens=4)
    common.seq_lens_cpu_upper_bound = torch.tensor([700, 9000, 33, 4])  # three decodes, then the prefill request
    assert b.build(0, common).decode.seq_lens_host == [700, 9000, 33]
    assert b.build_for_cudagraph_capture(common).decode.seq_lens_host is None
    plain = _metadata(num_decodes=2)
    assert b.build(0, plain).decode.seq_lens_host is None
    monkeypatch.setenv("RESIDUE_ATTN_CG_CAPTURE_LEN", "512")
    assert Bld(None, [], cfg, "cpu")._cg_capture_seq_len == 512
    with pytest.raises(NotImplementedError):
        b.build(0, _metadata(cascade=True))


# ------------------------------------------------------------------------------------------- the implementation
def _stock_init(self, num_heads, head_size, scale, num_kv_heads, alibi_slopes=None, sliding_window=None,
                kv_cache_dtype="nvfp4", logits_soft_cap=None, attn_type=None, kv_sharing_target_layer_name=None,
                sinks=None):
    """The attributes ``FlashInferImpl.__init__`` leaves behind, without its platform queries."""
    self.num_heads, self.head_size, self.scale, self.num_kv_heads = num_heads, head_size, float(scale), num_kv_heads
    self.alibi_slopes = alibi_slopes
    self.window_left = -1 if sliding_window is None else sliding_window - 1
    self.kv_cache_dtype = kv_cache_dtype
    self.is_kvcache_nvfp4 = kv_cache_dtype == "nvfp4"
    self.logits_soft_cap = logits_soft_cap
    self.kv_sharing_target_layer_name = kv_sharing_target_layer_name
    self.sinks = sinks
    self.supports_quant_query_input = True


@pytest.fixture()
def impl_cls(monkeypatch):
    from vllm.v1.attention.backends.flashinfer import FlashInferBackend, FlashInferImpl
    from resinfer_b200.quant.vllm_integration.attn import backend
    monkeypatch.setattr(FlashInferImpl, "__init__", _stock_init)
    monkeypatch.setattr(FlashInferBackend, "get_kv_cache_stride_order", staticmethod(lambda *a, **k: (0, 1, 3, 2, 4)))
    return backend.ResAttnFlashInferImpl


def test_constructor_keeps_bf16_queries_and_refuses_what_the_kernel_lacks(impl_cls):
    from vllm.model_executor.layers.quantization.utils.quant_utils import kFp8StaticTensorSym, kNvfp4Dynamic
    from resinfer_b200.quant.vllm_integration.attn import warmup
    impl = impl_cls(32, 128, 0.088, 8)
    assert impl.supports_quant_query_input is False and impl._decode_reduction_workspaces == {}
    assert impl.fused_output_quant_supported(kNvfp4Dynamic) and not impl.fused_output_quant_supported(kFp8StaticTensorSym)
    assert not impl_cls(32, 256, 0.06, 8).fused_output_quant_supported(kNvfp4Dynamic)
    assert (32, 8, 128, False) in warmup._DECODE_WARMUP_PROVIDER._geometries
    assert warmup._DECODE_WARMUP_PROVIDER.get_cutedsl_warmup_compile_units() == []       # no GPU here
    for args, kwargs in [((32, 128, 0.1, 8), dict(kv_cache_dtype="fp8")), ((32, 64, 0.1, 8), {}), ((32, 128, 0.1, 16), {}),
                         ((30, 128, 0.1, 8), {}), ((32, 128, 0.1, 0), {})]:
        with pytest.raises(NotImplementedError, match="NVFP4, D128/D256, and GQA4/6/8"):
            impl_cls(*args, **kwargs)
    for kwargs in [dict(alibi_slopes=[1.0]), dict(sliding_window=1024), dict(logits_soft_cap=30.0),
                   dict(sinks=torch.zeros(32)), dict(kv_sharing_target_layer_name="layer.3")]:
        with pytest.raises(NotImplementedError, match="Unsupported ResAttn decode"):
            impl_cls(32, 128, 0.1, 8, **kwargs)
    assert impl_cls(24, 128, 0.1, 4).num_heads == 24                                       # groups of six


def _vllm_cache(pages, page, hkv, d, seed=0):
    """vLLM's NVFP4 cache: logical [pages, 2, page, Hkv, 9 d / 16] over HND memory, every side of a page =
    its codes [Hkv, page, d/2] followed by its block scales [Hkv, page, d/16]."""
    g = torch.Generator().manual_seed(seed)
    full = d // 2 + d // 16
    mem = torch.randint(0, 256, (pages, 2, hkv, page, full), generator=g, dtype=torch.uint8)
    return mem.permute(0, 1, 3, 2, 4), mem


def test_pool_views_address_the_interleaved_cache_in_place(impl_cls):
    from resinfer_b200 import ops
    pages, page, hkv, d = 5, 16, 2, 128
    cache, mem = _vllm_cache(pages, page, hkv, d)
    layer = types.SimpleNamespace(_k_scale_float=0.5, _v_scale_float=0.25)
    impl = impl_cls(8, d, 0.1, hkv)
    pool = impl._pool_for(cache, layer)
    side = hkv * page * (d // 2 + d // 16)
    flat = mem.reshape(pages, 2, side)
    for which, (codes, sf) in enumerate(((pool.k_data, pool.k_sf), (pool.v_data, pool.v_sf))):
        assert codes.shape == (pages, hkv, page, d // 2) and sf.shape == (pages, hkv, page, d // 16)
        want_codes = flat[:, which, :hkv * page * d // 2].reshape(pages, hkv, page, d // 2)
        want_sf = flat[:, which, hkv * page * d // 2:].reshape(pages, hkv, page, d // 16)
        assert torch.equal(codes, want_codes) and torch.equal(sf.view(torch.uint8), want_sf)
        assert codes.data_ptr() == mem.data_ptr() + which * side                  # views, not copies
    assert (pool.page_size, pool.k_global_scale, pool.v_global_scale) == (page, 0.5, 0.25)
    assert ops.kv_page_strides(pool.k_data, pool.k_sf, pool.v_data, pool.v_sf) == (2 * side, 2 * side)
    assert impl._pool_for(cache, layer) is pool                                     # cached
    layer._v_scale_float = 0.125
    assert impl._pool_for(cache, layer) is not pool                                 # new scales: rebuilt
    with pytest.raises(ValueError, match="stock HND cache"):
        impl_cls(8, 256, 0.1, hkv)._pool_for(cache, layer)                          # head dimension of another model


def test_kv_page_strides_validation():
    from resinfer_b200 import ops
    kd = torch.zeros(4, 2, 16, 64, dtype=torch.uint8)
    ks = torch.zeros(4, 2, 16, 8, dtype=torch.uint8)
    assert ops.kv_page_strides(kd, ks, kd, ks) == (2 * 16 * 64, 2 * 16 * 8)
    with pytest.raises(ValueError, match="dense inner dimensions"):
        ops.kv_page_strides(kd.transpose(1, 2), ks, kd, ks)
    with pytest.raises(ValueError, match="same page strides"):
        ops.kv_page_strides(kd, ks, torch.zeros(4, 2, 2, 16, 64, dtype=torch.uint8)[:, 0], ks)
    with pytest.raises(ValueError, match="byte tensor"):
        ops.kv_page_strides(kd.to(torch.int16), ks, kd, ks)


def test_forward_checks_its_arguments(impl_cls):
    impl = impl_cls(32, 128, 0.1, 8)
    q = torch.zeros(4, 32, 128, dtype=torch.bfloat16)
    out = torch.ones(4, 32, 128, dtype=torch.bfloat16)
    assert impl.forward(None, q, None, None, None, None, out) is out and float(out.abs().sum()) == 0.0   # profiling run
    md = _metadata(num_decodes=4)
    with pytest.raises(ValueError, match="data and block scales"):
        impl.forward(None, q, None, None, None, md, out, output_scale=torch.ones(1))
    with pytest.raises(ValueError, match="BF16 Q"):
        impl.forward(None, q.to(torch.float8_e4m3fn), None, None, None, md, out)
    with pytest.raises(ValueError, match="output dtype"):
        impl.forward(None, q, None, None, None, md, out, output_scale=torch.ones(1), output_block_scale=torch.ones(1))
    with pytest.raises(ValueError, match="output dtype"):
        impl.forward(None, q, None, None, None, md, out.view(torch.uint8))
    md.decode = types.SimpleNamespace()                                             # not the TRTLLM form
    with pytest.raises(NotImplementedError, match="TRTLLM_GEN decode"):
        impl.forward(None, q, None, None, None, md, out)


def test_forward_divides_a_mixed_step_between_stock_prefill_and_resattn_decode(impl_cls, monkeypatch):
    from vllm.v1.attention.backends.flashinfer import FlashInferImpl
    calls = []

    def stock_forward(self, layer, query, key, value, kv_cache, md, output, output_scale=None, output_block_scale=None):
        calls.append(("prefill", query.dtype, tuple(query.shape), md.num_actual_tokens, md.num_decodes, md.decode,
                      md.slot_mapping.tolist(), tuple(key.shape)))
        output.fill_(2.0)
        return output
    monkeypatch.setattr(FlashInferImpl, "forward", stock_forward)
    impl = impl_cls(8, 128, 0.1, 2)
    monkeypatch.setattr(impl, "_pool_for", lambda kv, layer: "pool")

    def decode(q, pool, md, out3):
        calls.append(("decode", q.dtype, tuple(q.shape), q.is_contiguous(), pool, md.num_decode_tokens))
        out3[:md.num_decode_tokens].fill_(1.0)
    monkeypatch.setattr(impl, "_decode_forward", decode)
    layer = types.SimpleNamespace(_q_scale_float=0.5)
    n_dec, n_pre = 3, 5
    md = _metadata(num_decodes=n_dec, num_prefill_tokens=n_pre)
    qkv = torch.randn(n_dec + n_pre + 2, 3, 8 * 128).to(torch.bfloat16)            # two padding tokens at the end
    q = qkv[:, 0].view(-1, 8, 128)                                                  # strided like vLLM's split
    k = torch.zeros(n_dec + n_pre + 2, 2, 128, dtype=torch.bfloat16)
    out = torch.zeros(n_dec + n_pre + 2, 8, 128, dtype=torch.bfloat16)
    assert impl.forward(layer, q, k, k, None, md, out) is out
    pre, dec = calls
    # prefill: tokens after the decodes, FP8 as the stock metadata asks, its own slots, no decode part
    assert pre[:6] == ("prefill", torch.float8_e4m3fn, (n_pre, 8, 128), n_pre, 0, None)
    assert pre[6] == list(range(n_dec, n_dec + n_pre)) and pre[7] == (n_pre, 2, 128)
    assert dec == ("decode", torch.bfloat16, (n_dec, 8, 128), True, "pool", n_dec)
    assert float(out[:n_dec].min()) == 1.0 and float(out[n_dec:n_dec + n_pre].min()) == 2.0
    assert float(out[n_dec + n_pre:].abs().sum()) == 0.0                            # padding untouched
    assert md.num_decodes == n_dec and md.decode is not None                        # caller's metadata unchanged

    # the FP8 prefill query is the BF16 one divided by the layer's query scale
    calls.clear()
    seen = {}

    def stock_forward2(self, layer, query, key, value, kv_cache, md, output, *a, **k):
        seen["q"] = query
        return output
    monkeypatch.setattr(FlashInferImpl, "forward", stock_forward2)
    md2 = _metadata(num_decodes=0, num_prefill_tokens=4)
    q2 = (torch.randn(4, 8, 128) * 3).to(torch.bfloat16)
    impl.forward(layer, q2, k[:4], k[:4], None, md2, out[:4])
    assert torch.equal(seen["q"], (q2.float() * 2.0).clamp(-448, 448).to(torch.float8_e4m3fn))

    # decode only
    calls.clear()
    md3 = _metadata(num_decodes=4)
    impl.forward(layer, q2, k[:4], k[:4], None, md3, out[:4])
    assert [c[0] for c in calls] == ["decode"]
    # decode only, fused NVFP4 output: the packed variant of the mixin
    packed = []
    monkeypatch.setattr(impl, "_decode_forward_nvfp4", lambda q, pool, md, o, s, bs: packed.append((o.dtype, s, bs)))
    o8 = torch.zeros(4, 8 * 64, dtype=torch.uint8)
    impl.forward(layer, q2, k[:4], k[:4], None, md3, o8, output_scale="gs", output_block_scale="bs")
    assert packed == [(torch.uint8, "gs", "bs")]
    # mixed step with fused output: BF16 scratch for both halves, then one quantiser call over all tokens
    quant = []
    monkeypatch.setattr(impl, "_pack_nvfp4", lambda bf16, n, o, s, bs: quant.append((bf16.dtype, tuple(bf16.shape), n, s, bs)))
    monkeypatch.setattr(FlashInferImpl, "forward", stock_forward)
    calls.clear()
    o8 = torch.zeros(n_dec + n_pre + 2, 8 * 64, dtype=torch.uint8)
    impl.forward(layer, q, k, k, None, md, o8, output_scale="gs", output_block_scale="bs")
    assert [c[0] for c in calls] == ["prefill", "decode"]
    assert quant == [(torch.bfloat16, tuple(q.shape), n_dec + n_pre, "gs", "bs")]


def test_warmup_provider_lists_one_unit_per_head_dim(monkeypatch):
    from resinfer_b200.nvfp4.cute_attn import host
    from resinfer_b200.quant.vllm_integration.attn import runtime, warmup
    specs = host.decode_compile_variants(32, 8, 128, residue_fold=True, output_nvfp4=False)
    assert [s["args"] for s in specs] == [(128,)] and specs[0]["label"] == "D128"
    with pytest.raises(NotImplementedError):
        host.decode_compile_variants(32, 8, 128, residue_fold=False, output_nvfp4=False)
    with pytest.raises(NotImplementedError):
        runtime._validate_residue_geometry(32, 16)
    runtime._validate_residue_geometry(48, 8)
    prov = warmup._DecodeWarmupProvider()
    prov.add_geometry(32, 8, 128, True)
    prov.add_geometry(64, 8, 128, False)
    prov.add_geometry(32, 8, 256, False)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(warmup, "_load_decode_kernel", lambda: host)
    units = prov.get_cutedsl_warmup_compile_units()
    assert sorted(u.name for u in units) == ["resattn_decode[D128]", "resattn_decode[D256]"]     # duplicates folded
