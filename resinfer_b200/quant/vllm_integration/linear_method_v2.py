"""Residue NVFP4 linear method for vLLM: ``create_weights`` / ``process_weights_after_loading`` / ``apply`` of a
ModelOpt-NVFP4 checkpoint with residue metadata, on top of ``torch.ops.residue.nvfp4_linear``.

Interface and per-layer state follow the reference's quant/vllm_integration/linear_method_v2.py:105-618:

* three runtime modes read from ``residue_kernel_metadata.json``: ``standard`` (plain NVFP4), ``extended_k`` (weight
  ``[W | W[:, sel]]`` over K + S, activation residues appended along K) and ``mext_r1`` (weight at K, every channel
  carries a residue, applied at every M);
* the checkpoint contract is vLLM's ModelOpt NVFP4 one (``weight`` uint8 [N, K/2], ``weight_scale`` E4M3 [N, K/16],
  ``weight_scale_2``, ``input_scale``) with the input width replaced by the extended K of the layer; the salient
  indices arrive either as the checkpoint tensor ``<layer>.input_quantizer._salient_indices`` or from the sidecar;
* row-parallel layers cut the extended K with ``ResidueShardPlan`` and get their loaders wrapped so that the stock
  contiguous narrow lands on this rank's [base | salient] ranges;
* after loading: global scales -> ``alpha`` and ``input_global_scale_inv``, block scales -> 128x4 swizzle, channel
  mask from the (rank-local) indices, and -- with ``RESIDUE_ENABLE_DECODE_MEXT=1`` -- the base-K scale buffer that
  makes the layer fold-eligible at decode sizes.

What differs from the reference, by design of this library: there is no second NVFP4 backend underneath, so plain
layers run through the same op (its ``plain`` / fold routes) instead of a vLLM kernel object, and the class works
against the installed vLLM (its ``ModelOptNvFp4LinearMethod`` is the base class when importable) as well as
without vLLM at all (parameters are then plain ``torch.nn.Parameter`` objects with ``weight_loader`` /
``input_dim`` / ``output_dim`` attributes, which is what the unit tests drive).
"""
from __future__ import annotations

import torch
from torch.nn.parameter import Parameter

from . import residue_linear_op  # noqa: F401  (registers residue::nvfp4_linear)
from .env_contract import settings
from .metadata import get_extended_dim, get_layer_metadata
from .residue_tp import SF_VEC_SIZE, current_tp_rank, interleave_extended_for_tp, plan_from_partition
from .util import prepare_decode_mext_scale, swizzle_blockscale

try:                                                        # the installed vLLM, when there is one
    from vllm.model_executor.layers.quantization.modelopt import ModelOptNvFp4LinearMethod as _VllmBase
except Exception:                                           # no vLLM (or one that cannot be imported here)
    _VllmBase = None


def _vllm_parallel_state_ready() -> bool:
    try:
        from vllm.distributed.parallel_state import model_parallel_is_initialized
        return bool(model_parallel_is_initialized())
    except Exception:
        return False


class _InputQuantizerState(torch.nn.Module):
    """Receives the checkpoint tensor ``<layer>.input_quantizer._salient_indices``."""

    def __init__(self):
        super().__init__()
        self.register_buffer("_salient_indices", torch.empty(0, dtype=torch.int64))


def _plain_parameter(data: torch.Tensor, weight_loader, **attrs) -> Parameter:
    p = Parameter(data, requires_grad=False)
    p.weight_loader = weight_loader if weight_loader is not None else _copy_loader
    for k, v in attrs.items():
        setattr(p, k, v)
    return p


def _copy_loader(param, loaded_weight, *args, **kwargs):
    """Loader of the vLLM-free parameters: the tensor this rank needs is the leading part of ``loaded_weight``
    along the input dimension (the interleave put it there), everything else is copied whole."""
    dim = getattr(param, "input_dim", None)
    if dim is not None and loaded_weight.shape[dim] != param.shape[dim]:
        rank = int(getattr(param, "tp_rank", 0))
        loaded_weight = loaded_weight.narrow(dim, rank * param.shape[dim], param.shape[dim])
    param.data.copy_(loaded_weight.reshape(param.shape))


_Base = _VllmBase if _VllmBase is not None else object


class ResidueNvFp4LinearMethodV2(_Base):
    """See the module docstring.  One instance per layer (``layer_prefix`` names it)."""

    MODE_STANDARD = "standard"
    MODE_MEXT_R1 = "mext_r1"
    MODE_EXTENDED_K = "extended_k"

    def __init__(self, quant_config, layer_prefix: str = ""):
        # the base class would pick one of vLLM's NVFP4 backends here; this method needs none
        self.quant_config = quant_config
        self.marlin_input_dtype = None
        self.layer_prefix = layer_prefix
        self.group_size = int(getattr(quant_config, "group_size", 16))
        self._settings = settings()

    # ------------------------------------------------------------------------------------------ mode
    def _runtime_mode(self, layer_name: str) -> str:
        meta = get_layer_metadata(self.quant_config, layer_name)
        if meta:
            return meta.get("runtime_mode", self.MODE_EXTENDED_K)      # sidecars older than the mode field
        if self._settings.mode == "mext_r1" and any(layer_name.endswith(p) for p in self._settings.projections):
            return self.MODE_MEXT_R1
        return self.MODE_STANDARD

    def _extended_dim(self, layer_name: str) -> int | None:
        if self._runtime_mode(layer_name) == self.MODE_MEXT_R1:         # the residue lives in M, the weight stays at K
            return None
        return get_extended_dim(self.quant_config, layer_name)

    # ------------------------------------------------------------------------------- create_weights
    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs):
        name = getattr(layer, "prefix", "") or self.layer_prefix
        extended = self._extended_dim(name)
        plan = None
        if extended is not None:
            meta = get_layer_metadata(self.quant_config, name) or {}
            row_parallel = input_size_per_partition < input_size
            plan = plan_from_partition(extended_dim=extended, input_size_per_partition=input_size_per_partition,
                                       input_size=input_size, num_salient=int(meta.get("num_salient", 0)),
                                       tp_rank=current_tp_rank() if row_parallel else 0)
            input_size_per_partition = plan.k_ext_shard if plan is not None else extended
            input_size = extended
        self._create_nvfp4_parameters(layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                                      params_dtype, **extra_weight_attrs)
        if plan is not None:
            layer._residue_shard_plan = plan
            self._wrap_extended_loaders(layer, plan)
        layer.register_module("input_quantizer", _InputQuantizerState())
        layer._is_residue_layer = False
        layer.num_salient = 0

    def _create_nvfp4_parameters(self, layer, k_part, out_parts, k_full, n_full, params_dtype, **extra):
        if k_part % 16:
            raise ValueError(f"input size per partition must be a multiple of 16, got {k_part}")
        if _VllmBase is not None and _vllm_parallel_state_ready():
            _VllmBase.create_weights(self, layer, k_part, out_parts, k_full, n_full, params_dtype, **extra)
            return
        n_part = sum(out_parts)
        loader = extra.get("weight_loader")
        layer.logical_widths = list(out_parts)
        layer.input_size_per_partition = k_part
        layer.output_size_per_partition = n_part
        layer.params_dtype = params_dtype
        rank = int(extra.get("tp_rank", 0))
        layer.register_parameter("weight", _plain_parameter(
            torch.empty(n_part, k_part // 2, dtype=torch.uint8), loader, input_dim=1, output_dim=0, tp_rank=rank))
        layer.register_parameter("input_scale", _plain_parameter(
            torch.empty(len(out_parts), dtype=torch.float32), loader))
        layer.register_parameter("weight_scale_2", _plain_parameter(
            torch.empty(len(out_parts), dtype=torch.float32), loader))
        layer.register_parameter("weight_scale", _plain_parameter(
            torch.empty(n_part, k_part // self.group_size, dtype=torch.float8_e4m3fn), loader,
            input_dim=1, output_dim=0, tp_rank=rank))

    @staticmethod
    def _wrap_extended_loaders(layer, plan) -> None:
        """Reorder the checkpoint's [base | salient] columns into per-rank [base_r | salient_r] runs before the
        stock loader takes this rank's contiguous slice.  ``weight`` packs two channels per byte, ``weight_scale``
        holds one entry per 16 channels; tensors of any other width are not K-extended and pass through."""
        for pname, per_element in (("weight", 2), ("weight_scale", SF_VEC_SIZE)):
            param = getattr(layer, pname, None)
            inner = getattr(param, "weight_loader", None) if param is not None else None
            if inner is None:
                continue

            def loader(p, loaded, *args, _inner=inner, _per=per_element, **kwargs):
                if loaded.shape[-1] == plan.k_ext // _per:
                    loaded = interleave_extended_for_tp(loaded, plan, channels_per_element=_per)
                return _inner(p, loaded, *args, **kwargs)

            try:
                param.weight_loader = loader
            except AttributeError:                          # vLLM parameters expose the loader read-only
                param._weight_loader = loader

    # ------------------------------------------------------------- process_weights_after_loading
    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        name = getattr(layer, "prefix", "") or self.layer_prefix
        mode = self._runtime_mode(name)
        layer._runtime_mode = mode
        dev = layer.weight.device
        indices = None
        if mode != self.MODE_MEXT_R1:
            got = layer.input_quantizer._salient_indices if hasattr(layer, "input_quantizer") else None
            if got is not None and got.numel() > 0:
                indices = got.to(dev)
            else:
                meta = get_layer_metadata(self.quant_config, name)
                if meta and meta.get("salient_indices"):
                    indices = torch.tensor(meta["salient_indices"], dtype=torch.int64, device=dev)
            plan = getattr(layer, "_residue_shard_plan", None)
            if plan is not None and indices is not None:
                indices = plan.local_salient_indices(indices)         # this rank's channels, rebased to its slice
        extended_in = layer.weight.shape[1] * 2
        layer.extended_in_features = extended_in
        layer._salient_indices = indices if indices is not None and indices.numel() else None
        layer.num_salient = 0 if layer._salient_indices is None else int(indices.numel())
        layer.original_in_features = extended_in - layer.num_salient
        layer._is_residue_layer = mode == self.MODE_MEXT_R1 or layer.num_salient > 0
        layer.channel_mask = None
        if layer.num_salient:
            from ...nvfp4.quant import indices_to_channel_masks
            layer.channel_mask = indices_to_channel_masks(layer._salient_indices, layer.original_in_features,
                                                          layer_name=name).to(dev)
        raw_scale = layer.weight_scale.data
        if raw_scale.dtype != torch.float8_e4m3fn:
            raise ValueError("weight block scales must be float8_e4m3fn")
        # one global scale per layer: merged projections (qkv, gate_up) share the largest of their parts
        in_gs = layer.input_scale.max().to(torch.float32)
        w_gs = layer.weight_scale_2.max().to(torch.float32)
        del layer.input_scale, layer.weight_scale_2
        layer.input_global_scale = Parameter(in_gs, requires_grad=False)
        layer.weight_global_scale = Parameter(w_gs, requires_grad=False)
        layer.alpha = Parameter((in_gs * w_gs).reshape(1), requires_grad=False)
        layer.input_global_scale_inv = Parameter((1.0 / in_gs).to(torch.float32).reshape(1), requires_grad=False)
        layer.weight = Parameter(layer.weight.data, requires_grad=False)
        layer.weight_scale = Parameter(swizzle_blockscale(raw_scale), requires_grad=False)
        layer.weights_padding_cols = 0
        layer._decode_mext_layout_enabled = False
        if mode == self.MODE_MEXT_R1:
            # the whole scale buffer is its own base-K prefix: the fold reads the entire weight
            layer.weight_scale_base = layer.weight_scale
            layer._mext_decode_k_base = int(extended_in)
            layer._decode_mext_layout_enabled = True
        elif self._settings.decode_mext:
            if layer.num_salient:
                prepare_decode_mext_scale(layer, raw_scale)          # from the RAW scale: a swizzled one cannot be sliced
            else:
                layer.weight_scale_base = layer.weight_scale          # plain layer: the fold is a free precision bonus at small M
                layer._mext_decode_k_base = int(layer.original_in_features)
                layer._decode_mext_layout_enabled = True
        if not hasattr(layer, "weight_scale_base"):
            layer.weight_scale_base = layer.weight_scale              # placeholder the op ignores

    # ------------------------------------------------------------------------------------- apply
    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        n_out = int(layer.output_size_per_partition)
        out_shape = [*x.shape[:-1], n_out]
        x2d = x.reshape(-1, x.shape[-1]).contiguous()
        if x2d.shape[0] == 0:
            y = x2d.new_empty((0, n_out))
            return (y + bias if bias is not None else y).view(*out_shape)
        fold = bool(getattr(layer, "_decode_mext_layout_enabled", False))
        mask = layer.channel_mask if layer.channel_mask is not None else x2d.new_zeros(1, dtype=torch.uint8)
        y = torch.ops.residue.nvfp4_linear(
            x2d, layer.weight, layer.input_global_scale_inv, layer.weight_scale, layer.weight_scale_base, mask, layer.alpha,
            int(layer._mext_decode_k_base) if fold else 0, int(layer.num_salient), int(layer.weights_padding_cols), n_out,
            fold, False, layer._runtime_mode == self.MODE_MEXT_R1)
        if bias is not None:
            y = y + bias
        return y.view(*out_shape)
