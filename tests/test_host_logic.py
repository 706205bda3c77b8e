"""Host-side logic that needs no GPU: registry, routing, environment contract, split plans,
shard plans, wrappers' argument errors, weight preparation, plugin gates."""
import os

import numpy as np
import pytest
import torch

import oracle as O


# ---------------------------------------------------------------------------------- registry
def test_linear_registry_contract():
    from resinfer_b200.quant.linear_registry import LinearRegistry, TorchLinearWrapper
    import resinfer_b200.quant.linear_impls  # noqa: F401
    assert {"TorchLinear", "ResidueLinear", "ResidueSwapLinear", "NVFP4Linear"} <= set(LinearRegistry.list())
    assert LinearRegistry.get("TorchLinear") is TorchLinearWrapper
    lin = torch.nn.Linear(8, 8)
    assert TorchLinearWrapper.from_linear(lin) is lin
    with pytest.raises(KeyError, match="not registered"):
        LinearRegistry.get("nope")
    with pytest.raises(TypeError, match="from_linear"):
        @LinearRegistry.register("bad")
        class Bad(torch.nn.Module):
            pass
    assert not LinearRegistry.is_registered("bad")
    saved = dict(LinearRegistry._registry)
    LinearRegistry.clear()
    assert LinearRegistry.list() == []
    LinearRegistry._registry.update(saved)


# ---------------------------------------------------------------------------------- routing
def test_route_thresholds():
    from resinfer_b200.quant.vllm_integration.residue_linear_op import _route
    kw = dict(arch="sm100", fold_max_m=128, ratio1_fold_max_m=512, force_fold=False)
    assert _route(1, fold_eligible=True, ratio1=True, num_salient=0, **kw) == "sm10x_fold"
    assert _route(512, fold_eligible=True, ratio1=True, num_salient=0, **kw) == "sm10x_fold"
    assert _route(513, fold_eligible=True, ratio1=True, num_salient=0, **kw) == "ratio1_prefill"
    assert _route(128, fold_eligible=True, ratio1=False, num_salient=640, **kw) == "sm10x_fold"
    assert _route(129, fold_eligible=True, ratio1=False, num_salient=640, **kw) == "k_ext"
    assert _route(129, fold_eligible=True, ratio1=False, num_salient=0, **kw) == "plain"
    assert _route(4, fold_eligible=False, ratio1=True, num_salient=0, **kw) == "invalid_mext"
    kw["arch"] = None
    assert _route(4, fold_eligible=True, ratio1=False, num_salient=640, **kw) == "k_ext"


def test_env_contract():
    from resinfer_b200.quant.vllm_integration.env_contract import parse_settings
    s = parse_settings({})
    assert s.mode == "v2" and s.decode_max_m is None and s.ratio1_prefill == "auto" and "o_proj" in s.projections
    s = parse_settings({"RESIDUE_PATCH_MODE": "MEXT-R1", "RESIDUE_DECODE_MEXT_MAX_M": "64", "RESIDUE_FORCE_DECODE_MEXT": "1"})
    assert s.mode == "mext_r1" and s.decode_max_m == 64 and s.force_fold
    for bad in ({"RESIDUE_PATCH_MODE": "v3"}, {"RESIDUE_FORCE_DECODE_MEXT": "yes"}, {"RESIDUE_MEXT_FOLD_MAX_M": "-1"},
                {"RESIDUE_RATIO1_PREFILL_PATH": "x"}):
        with pytest.raises(ValueError):
            parse_settings(bad)


# ---------------------------------------------------------------------------------- attention plan
def test_decode_plan_selection_and_validation():
    from resinfer_b200.nvfp4.cute_attn.plan import select_decode_plan, validate_decode_plan, static_compile_plans
    assert select_decode_plan(256, 8, 32768, 148, head_dim=256) == (1, "none")
    # a handful of (sequence, KV head) pairs: the splits form a cluster, one CTA per SM
    assert select_decode_plan(1, 8, 16384, 148) == (8, "cga_sharded")
    s, r = select_decode_plan(1, 8, 32768, 148)                            # very long: more ticket splits win
    assert r == "kernel" and 8 <= s <= 64
    assert select_decode_plan(1, 8, 4096, 148) == (8, "cga_sharded")
    assert select_decode_plan(1, 8, 4096, 148, head_dim=256) == (8, "cga_sharded")
    assert select_decode_plan(1, 8, 600, 148) == (5, "cga_sharded")        # one split per tile at most
    assert select_decode_plan(4, 2, 8192, 148) == (8, "cga_sharded")       # a tensor-parallel shard's heads
    assert select_decode_plan(1, 32, 8192, 148)[1] == "kernel"             # too many clusters
    s, r = select_decode_plan(1, 8, 32768, 148, reduction_policy="deterministic")
    assert r == "kernel" and 8 <= s <= 64
    s, r = select_decode_plan(1, 8, 32768, 148, output_nvfp4=True)         # packed output: ticket reducer
    assert r == "kernel" and 8 <= s <= 64
    # eight sequences of up to 32768 tokens: pieces sized so that the working CTAs fill the SMs once
    assert select_decode_plan(8, 8, 32768, 148, head_dim=256) == (4, "kernel")
    assert select_decode_plan(8, 8, 32768, 148) == (8, "kernel")       # head_dim 128: two CTAs per SM
    assert select_decode_plan(64, 8, 32768, 148) == (3, "kernel")     # a few waves: thirds even out the tail
    assert select_decode_plan(1, 8, 64, 148) == (1, "none")          # too short to split
    # lengths known on the host, small grid: the most splits whose working CTAs fit the device once
    assert select_decode_plan(4, 8, 32768, 148, seq_lens=[32768] * 4) == (9, "kernel")        # 288 of 296 slots
    assert select_decode_plan(8, 8, 32768, 148, seq_lens=[32768] * 8) == (4, "kernel")
    assert select_decode_plan(8, 8, 32768, 148, head_dim=256, seq_lens=[32768] * 8) == (2, "kernel")
    uneven = [2525, 19358, 12195, 15818, 10090, 9605, 25861, 5305]
    assert select_decode_plan(8, 8, 25861, 148, seq_lens=uneven) == (8, "kernel")             # short sequences leave splits unused
    assert select_decode_plan(2, 8, 8192, 148, seq_lens=[8192, 8192]) == (16, "kernel")        # 64 tiles: pieces of 4, no empty splits
    assert select_decode_plan(64, 8, 32768, 148, seq_lens=[32768] * 64) == select_decode_plan(64, 8, 32768, 148)   # large grids: unchanged
    assert select_decode_plan(8, 8, 32768, 148, seq_lens=[32768] * 7) == select_decode_plan(8, 8, 32768, 148)      # wrong count: ignored
    assert (1, "none") in static_compile_plans()
    validate_decode_plan((4, "kernel"))
    for bad in ((0, "kernel"), (2, "none"), (2, "magic"), (1024, "kernel")):
        with pytest.raises(ValueError):
            validate_decode_plan(bad)
    with pytest.raises(NotImplementedError):
        select_decode_plan(1, 8, 100, 148, head_dim=64)
    validate_decode_plan((4, "cga_sharded"), head_dim=256)
    validate_decode_plan((16, "cga_sharded"))
    with pytest.raises(NotImplementedError):
        validate_decode_plan((4, "gmem_fused"), head_dim=256)
    with pytest.raises(NotImplementedError):
        validate_decode_plan((4, "cga_sharded"), output_nvfp4=True)
    with pytest.raises(ValueError):
        validate_decode_plan((12, "cga_sharded"))
    assert (4, "cga_sharded") in static_compile_plans() and (4, "cga_sharded") not in static_compile_plans(output_nvfp4=True)
    with pytest.raises(ValueError):
        select_decode_plan(1, 8, 100, 148, reduction_policy="fastest")


def test_attention_shape_checks():
    from resinfer_b200.nvfp4.cute_attn.host import check_shape_supported, _residue_padded_group_size
    assert _residue_padded_group_size(32, 8) == 8 and _residue_padded_group_size(64, 8) == 16
    check_shape_supported(64, 8, 128)
    with pytest.raises(NotImplementedError):
        check_shape_supported(64, 8, 64)
    with pytest.raises(NotImplementedError):
        check_shape_supported(40, 8, 128)
    with pytest.raises(ValueError):
        check_shape_supported(65, 8, 128)
    with pytest.raises(NotImplementedError):
        check_shape_supported(64, 8, 128, prediction=2)


# ---------------------------------------------------------------------------------- TP shard plan
def test_shard_plan_ranges_and_gather():
    from resinfer_b200.quant.vllm_integration.residue_tp import (ResidueShardPlan, ResidueTPError,
                                                                  interleave_extended_for_tp, plan_from_partition)
    k, s, tp = 1024, 256, 4
    assert plan_from_partition(extended_dim=k + s, input_size_per_partition=k, input_size=k, num_salient=s) is None
    plan = plan_from_partition(extended_dim=k + s, input_size_per_partition=k // tp, input_size=k, num_salient=s, tp_rank=2)
    assert (plan.base_shard, plan.salient_shard, plan.k_ext_shard) == (256, 64, 320)
    assert plan.ranges() == ((512, 256), (k + 128, 64))
    assert plan.ranges(2) == ((256, 128), ((k + 128) // 2, 32))
    full = torch.arange(k + s)
    mine = plan.gather(full)
    assert mine.tolist() == list(range(512, 768)) + list(range(k + 128, k + 192))
    inter = interleave_extended_for_tp(full, plan)
    assert torch.equal(inter[2 * 320:3 * 320], mine) and sorted(inter.tolist()) == full.tolist()
    # salient indices: 2 per block of 8, globally sorted
    idx = torch.tensor(O.mask_to_indices(O.make_kext_mask(k, 2)))
    loc = plan.local_salient_indices(idx)
    assert loc.numel() == 64 and loc.min() >= 0 and loc.max() < 256
    with pytest.raises(ResidueTPError, match="sorted"):
        plan.local_salient_indices(idx.flip(0))
    with pytest.raises(ResidueTPError):
        plan.gather(torch.arange(k + s + 1))


def test_shard_plan_rejections_match_the_reference_rule():
    """The cells of the KEXT x TP grid that the reference's own rule accepts / rejects."""
    from resinfer_b200.quant.vllm_integration.residue_tp import ResidueTPError, plan_from_partition

    def ok(k, per8, tp, vec=16, blocks=4):
        s = k // 8 * per8
        try:
            plan_from_partition(extended_dim=k + s, input_size_per_partition=k // tp, input_size=k, num_salient=s,
                                scale_vec_size=vec, scale_swizzle_blocks=blocks)
            return True
        except ResidueTPError:
            return False

    for per8 in (1, 2, 4):
        for tp in (2, 4, 8):
            assert ok(8192, per8, tp)                      # o projection: every cell valid
    assert not ok(25600, 1, 4) and not ok(25600, 1, 8) and not ok(25600, 2, 8)     # down, NVFP4
    assert ok(25600, 1, 2) and ok(25600, 2, 4) and ok(25600, 4, 8)
    assert not ok(25600, 1, 8, vec=32, blocks=1) and ok(25600, 1, 4, vec=32, blocks=1)   # MXFP4
    with pytest.raises(ResidueTPError, match="does not match"):
        plan_from_partition(extended_dim=100, input_size_per_partition=32, input_size=64, num_salient=8)


# ---------------------------------------------------------------------------------- wrappers
def test_wrapper_argument_errors_before_launch():
    from resinfer_b200.nvfp4 import mext, quant
    from resinfer_b200.nvfp4.mxfp4 import selective
    x = torch.zeros(4, 24, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="multiple of 16"):
        mext.scaled_fp4_quant_mext_r1(x, torch.ones(1), layout_mode="row_pair", enable_pdl=False)
    x = torch.zeros(4, 32, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="divisible by 8"):
        mext.scaled_fp4_quant_mext_r1(x, torch.ones(1), layout_mode="tile8", enable_pdl=False)
    with pytest.raises(ValueError, match="only with tile8"):
        mext.scaled_fp4_quant_mext_r1(x, torch.ones(1), layout_mode="concat", m_pad_multiple=8, enable_pdl=False)
    with pytest.raises(ValueError, match="layout_mode"):
        mext.scaled_fp4_quant_mext_r1(x, torch.ones(1), layout_mode="zigzag", enable_pdl=False)
    with pytest.raises(ValueError, match="elts_mode"):
        mext.scaled_fp4_quant_mext_r1(x, torch.ones(1), elts_mode=12, enable_pdl=False)
    with pytest.raises(ValueError, match="Unsupported salient ratio"):
        quant._residue_per_8(100, 256)
    assert quant._residue_per_8(64, 256) == 2
    m = quant.indices_to_channel_masks(torch.tensor([0, 9, 23]), 24)
    assert m.tolist() == [1, 2, 128]
    idx, masks = selective.prepare_indices([1, 8, 17, 30], 32, "cpu")
    assert masks.tolist() == [2, 1, 2, 64] and idx.dtype == torch.int32
    for bad in ([1, 2, 17, 30], [8, 1, 17, 30], [1, 8, 17, 40]):
        with pytest.raises(ValueError):
            selective.prepare_indices(bad, 32, "cpu")
    with pytest.raises(ValueError, match="ratios"):
        selective.prepare_indices([1, 8, 17], 32, "cpu")


def test_weight_prep_matches_oracle_layout():
    from resinfer_b200.quant import weight_prep as wp
    w = torch.from_numpy(O.make_weight(200, 512))
    d = wp.quantize_weight_nvfp4(w)
    gs = np.float32(np.abs(w.numpy()).max() / (6 * 448))
    oc, osf = O.nvfp4_quant_plain(w.numpy(), np.float32(1) / gs)
    assert (d["weight"].numpy() == oc).mean() > 0.99 and (d["weight_scale"].numpy() == osf).mean() > 0.99
    assert d["weight_scale"].numel() == 2 * 8 * 512
    mx = wp.quantize_weight_mxfp4(w)
    oc, osf = O.mxfp4_quant_plain(w.numpy())
    assert np.array_equal(mx["weight"].numpy(), oc) and np.array_equal(mx["weight_scale"].numpy(), osf)
    idx = wp.salient_indices_per8(512, 2)
    ext = wp.quantize_weight_nvfp4(w, idx)
    assert ext["weight"].shape == (200, (512 + 128) // 2) and ext["num_salient"] == 128
    assert torch.equal(ext["weight"][:, :256], d["weight"])      # base prefix unchanged by the extension
    lin = torch.from_numpy(np.random.default_rng(0).integers(0, 255, (130, 10), dtype=np.uint8))
    assert np.array_equal(wp.swizzle_scales_any(lin).numpy(), O.swizzle_scales(lin.numpy()))


# ---------------------------------------------------------------------------------- plugin
def test_plugin_gates(monkeypatch, capsys):
    from resinfer_b200.runtime.vllm_plugin import residue_vllm_plugin as plug
    for k in ("RESIDUE_NVFP4", "RESIDUE_ATTN", "RESIDUE_MXFP4"):
        monkeypatch.delenv(k, raising=False)
    plug.apply()
    assert capsys.readouterr().out == ""                  # no gate, nothing happens
    monkeypatch.setenv("RESIDUE_MXFP4", "1")
    plug.apply()
    assert "applied" in capsys.readouterr().out
    assert hasattr(torch.ops.residue, "mxfp4_linear")
    import sys
    assert "nvfp4" in sys.modules and "quant.linear_registry" in sys.modules


def test_plugin_fails_closed(monkeypatch, capsys):
    from resinfer_b200.nvfp4 import extension
    from resinfer_b200.runtime.vllm_plugin import residue_vllm_plugin as plug
    monkeypatch.setenv("RESIDUE_NVFP4", "1")

    def boom(required=True):
        raise ImportError("native library missing")

    monkeypatch.setattr(extension, "ensure_loaded", boom)
    with pytest.raises(ImportError):
        plug.apply()
    assert "refusing to serve" in capsys.readouterr().out


def test_gemm_plan_selection_needs_no_gpu():
    """The library plans without a device (a 148-SM part is assumed): the measured table for the benchmark
    model's projections, the cost model elsewhere, no work for zero tokens."""
    from resinfer_b200.nvfp4.cute_fold.tactics import describe_plan, kernel_arch_for_capability
    assert kernel_arch_for_capability(10, 0) == "sm100" and kernel_arch_for_capability(12, 0) is None
    assert [describe_plan(m, 10240, 5120)["k_split"] for m in (1, 16, 128)] == [1, 1, 1]          # qkv: whole tiles
    assert [describe_plan(m, 5120, 8192)["k_split"] for m in (1, 16, 64)] == [3, 3, 2]            # o: 3 K slices, 2 above 16 tokens
    assert describe_plan(1, 51200, 5120)["k_split"] == 1 and describe_plan(64, 51200, 5120)["k_split"] == 1   # gate_up: whole tiles
    assert describe_plan(1, 5120, 25600)["workspace_bytes"] > 0                                   # K split -> scratch
    assert describe_plan(1024, 10240, 5120, layout="concat_k") == {"k_split": 1, "workspace_bytes": 0}
    assert describe_plan(0, 10240, 5120) == {"k_split": 1, "workspace_bytes": 0}
    assert describe_plan(16, 1280, 5120)["k_split"] > 1                                           # 10 tiles: split K
    assert describe_plan(16, 5120, 2048)["k_split"] == 1                                          # 40 tiles, short K: whole tiles
