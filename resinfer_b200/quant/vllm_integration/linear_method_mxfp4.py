"""MXFP4 linear method for vLLM: packed uint8 weights and E8M0 scales of a ModelOpt MXFP4 checkpoint, loaded per rank
and run by ``torch.ops.residue.mxfp4_linear``.

Interface, checks and error texts follow the reference's quant/vllm_integration/linear_method_mxfp4.py:105-276
(``ResidueMxfp4LinearMethod``) and :22-102 (``ModelOptMxfp4Config``, registered as ``modelopt_mxfp4`` when vLLM is
importable): K % 128 == 0 and N % 32 == 0 per rank; the sidecar record of the layer decides the mode (``standard``,
``selective`` over the K extension padded to 128, ``mext_r1``); tensor-parallel loading is opt-in
(``RESIDUE_MXFP4_TP_EXPERIMENTAL=1``), row-parallel selective layers interleave their extended columns before the
stock loader slices them; after loading the raw E8M0 scales are swizzled, the rank-local indices and masks built and
scale code 255 (NaN) rejected.
"""
from __future__ import annotations

import os

import torch
from torch.nn import Parameter

from .. import mxfp4_linear as _op  # noqa: F401  (registers residue::mxfp4_linear)
from ..kernel_metadata import padded_k, residue_spec
from .residue_tp import current_tp_rank, interleave_extended_for_tp, plan_from_partition

try:
    from vllm.model_executor.layers.linear import LinearMethodBase as _Base
except Exception:
    _Base = object


class ResidueMxfp4LinearMethod(_Base):
    def __init__(self, metadata=None, *, extended_dim=None):
        self.metadata = metadata or {}
        self.extended_dim = extended_dim

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra_weight_attrs):
        n, k = sum(output_partition_sizes), input_size_per_partition
        if params_dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("MXFP4 output dtype must be fp16 or bf16")
        if k <= 0 or k % 128 or n <= 0 or n % 32:
            raise ValueError("MXFP4 rank-local linear requires positive K%128==0 and N%32==0")
        # the sidecar describes the whole checkpoint, the parameters this rank's partition
        self.spec = residue_spec(self.metadata, input_size, output_size)
        self.mode = self.spec["mode"]
        self.indices = tuple(self.spec.get("indices", ()))
        if self.extended_dim is not None and self.extended_dim != padded_k(input_size, len(self.indices)):
            raise ValueError("metadata extended dimension does not match MXFP4 weights")
        row_parallel, column_parallel = k != input_size, n != output_size
        if (row_parallel or column_parallel) and os.environ.get("RESIDUE_MXFP4_TP_EXPERIMENTAL", "0") != "1":
            raise ValueError("MXFP4 TP loading is experimental; set RESIDUE_MXFP4_TP_EXPERIMENTAL=1 to opt in")
        if row_parallel and column_parallel:
            raise ValueError("MXFP4 cannot shard both input and output axes in one linear")
        if row_parallel and (k > input_size or input_size % k or output_size != n):
            raise ValueError("MXFP4 row-parallel partition does not match global shape")
        if column_parallel and (input_size != k or n > output_size):
            raise ValueError("MXFP4 column-parallel partition does not match global shape")
        plan = None
        if row_parallel and self.mode == "selective":
            plan = plan_from_partition(extended_dim=input_size + len(self.indices), input_size_per_partition=k,
                                       input_size=input_size, num_salient=len(self.indices), tp_rank=current_tp_rank(),
                                       scale_vec_size=32, scale_swizzle_blocks=1,      # checkpoint scales are linear
                                       k_alignment=128)
        kp = padded_k(k, plan.salient_shard if plan else len(self.indices))
        inner = extra_weight_attrs.pop("weight_loader", None) or _copy_loader
        layer._mxfp4_shard_plan = plan
        layer._mxfp4_loaded = {"weight": set(), "weight_scale": set()}
        layer._mxfp4_shards = len(output_partition_sizes)

        def checked(name, per_element):
            def load(param, tensor, *args, **kwargs):
                if tensor.dtype != torch.uint8:
                    raise ValueError(f"packed MXFP4 {name} must be uint8")
                if plan is not None:
                    tensor = interleave_extended_for_tp(tensor, plan, channels_per_element=per_element)
                inner(param, tensor, *args, **kwargs)
                shard = args[0] if args else kwargs.get("loaded_shard_id")
                if isinstance(shard, (tuple, list)):
                    layer._mxfp4_loaded[name].update(shard)
                else:
                    layer._mxfp4_loaded[name].add(shard)
            return load

        for name, width, per_element in (("weight", kp // 2, 2), ("weight_scale", kp // 32, 32)):
            param = Parameter(torch.empty(n, width, dtype=torch.uint8), requires_grad=False)
            for key, val in {"input_dim": 1, "output_dim": 0, **extra_weight_attrs,
                             "weight_loader": checked(name, per_element)}.items():
                setattr(param, key, val)
            layer.register_parameter(name, param)
        layer._mxfp4_input_size = k
        layer._mxfp4_output_dtype = params_dtype
        layer._mxfp4_prepared = False

    def process_weights_after_loading(self, layer):
        from ...nvfp4.mxfp4 import prepare_indices, swizzle_scales
        if layer._mxfp4_prepared:
            return
        weight = layer.weight.detach()
        if not weight.is_cuda or torch.cuda.get_device_capability(weight.device) != (10, 0):
            raise ValueError("MXFP4 weight preparation requires SM100")
        with torch.no_grad(), torch.cuda.device(weight.device):
            indices = torch.empty(0, dtype=torch.int32, device=weight.device)
            masks = torch.empty(0, dtype=torch.uint8, device=weight.device)
            if self.mode == "selective":
                selected = self.indices
                plan = layer._mxfp4_shard_plan
                if plan is not None:
                    selected = plan.local_salient_indices(torch.tensor(self.indices, dtype=torch.int32, device=weight.device))
                indices, masks = prepare_indices(selected, layer._mxfp4_input_size, weight.device)
            for name, loaded in layer._mxfp4_loaded.items():
                if None not in loaded and len(loaded) != layer._mxfp4_shards:
                    raise ValueError(f"incomplete packed MXFP4 {name} loading: {loaded}")
            if (layer.weight_scale == 255).any().item():
                raise ValueError("MXFP4 checkpoint contains NaN E8M0 scale code 255")
            scales = swizzle_scales(layer.weight_scale.detach().contiguous())
            del layer.weight_scale
            layer.weight = Parameter(weight, requires_grad=False)
            layer.register_buffer("weight_scale", scales)
            layer.register_buffer("salient_indices", indices)
            layer.register_buffer("salient_masks", masks)
            layer._mxfp4_prepared = True

    def apply(self, layer, x, bias=None):
        if not layer._mxfp4_prepared:
            raise RuntimeError("call process_weights_after_loading before MXFP4 apply")
        if x.shape[-1] != layer._mxfp4_input_size:
            raise ValueError("input feature dimension does not match loaded MXFP4 weight")
        return torch.ops.residue.mxfp4_linear(x, layer.weight, layer.weight_scale, layer.salient_indices,
                                              layer.salient_masks, self.mode, layer._mxfp4_output_dtype, bias)


def _copy_loader(param, tensor, *args, **kwargs):
    """Loader used when vLLM provides none (unit tests): this rank's leading slice along the input dimension."""
    dim = getattr(param, "input_dim", None)
    if dim is not None and tensor.shape[dim] != param.shape[dim]:
        tensor = tensor.narrow(dim, int(getattr(param, "tp_rank", 0)) * param.shape[dim], param.shape[dim])
    param.data.copy_(tensor)


def select_method(quant_config, prefix: str, is_layer_excluded):
    """The decision of ``ModelOptMxfp4Config.get_quant_method`` for a dense linear layer, apart from vLLM types:
    returns ``None`` for "leave unquantised", else a ``ResidueMxfp4LinearMethod``.  A fused runtime layer (qkv_proj,
    gate_up_proj) may be excluded as a whole or through ALL of its checkpoint constituents, never partly; its
    constituents must share one sidecar record and one extended width."""
    from .metadata import get_residue_metadata
    from ..kernel_metadata import get_fused_hf_candidates, get_residue_layer_candidates
    candidates = get_residue_layer_candidates(prefix)
    groups = get_fused_hf_candidates(prefix)
    if any(is_layer_excluded(name) for name in candidates):
        constituents = {name for group in groups for name in group}
        whole = any(is_layer_excluded(name) for name in candidates if name not in constituents)
        all_members = any(all(is_layer_excluded(name) for name in group) for group in groups)
        if not whole and not all_members:
            raise ValueError(f"partially quantized fused group: {prefix}")
        return None
    data = get_residue_metadata(quant_config, require_local=True)
    layers = data.get("layers", {})
    metas = [layers[name] for name in candidates if name in layers]
    if metas and any(meta != metas[0] for meta in metas[1:]):
        raise ValueError(f"fused group must share residue metadata: {prefix}")
    for names in groups:
        present = [name in layers for name in names]
        if any(present) and not all(present):
            raise ValueError(f"partially specified residue fused group: {prefix}")
    dims = data.get("extended_linear_dims", {})
    widths = {dims[name] for name in candidates if name in dims}
    if len(widths) > 1:
        raise ValueError(f"fused group must share extended input width: {prefix}")
    return ResidueMxfp4LinearMethod(metas[0] if metas else {}, extended_dim=next(iter(widths), None))


def parse_modelopt_mxfp4_config(config: dict) -> list:
    """Validate the ``quantization`` block of a ModelOpt MXFP4 checkpoint; returns its exclusion list."""
    quant = config.get("quantization", config)
    if str(quant.get("quant_algo", "")).upper() != "MXFP4":
        raise ValueError("ModelOpt MXFP4 adapter requires quant_algo=MXFP4")
    if quant.get("group_size", 32) != 32:
        raise ValueError("MXFP4 requires group_size=32")
    if quant.get("kv_cache_quant_algo") or quant.get("kv_cache_scheme"):
        raise ValueError("MXFP4 adapter does not support quantized KV cache")
    excluded = quant.get("exclude_modules", quant.get("ignore", []))
    if not isinstance(excluded, list) or any(not isinstance(v, str) for v in excluded):
        raise ValueError("ModelOpt exclude_modules/ignore must be a list of strings")
    return excluded


try:                                                        # the vLLM-facing config class, when vLLM is importable
    from vllm.model_executor.layers.linear import LinearBase, UnquantizedLinearMethod
    from vllm.model_executor.layers.quantization import register_quantization_config
    from vllm.model_executor.layers.quantization.modelopt import ModelOptQuantConfigBase

    @register_quantization_config("modelopt_mxfp4")
    class ModelOptMxfp4Config(ModelOptQuantConfigBase):
        """Native ModelOpt MXFP4 checkpoints; the residue part comes from the shared sidecar."""

        def __init__(self, exclude_modules=None):
            super().__init__(exclude_modules or [])

        @classmethod
        def get_name(cls):
            return "modelopt_mxfp4"

        @classmethod
        def get_supported_act_dtypes(cls):
            return [torch.float16, torch.bfloat16]

        @classmethod
        def get_min_capability(cls):
            return 100

        @classmethod
        def override_quantization_method(cls, hf_quant_cfg, user_quant, hf_config=None):
            return cls.get_name() if cls._extract_modelopt_quant_algo(hf_quant_cfg) == "MXFP4" else None

        @classmethod
        def from_config(cls, config):
            return cls(parse_modelopt_mxfp4_config(config))

        def get_quant_method(self, layer, prefix):
            try:
                from vllm.model_executor.layers.fused_moe import RoutedExperts
                if isinstance(layer, RoutedExperts):
                    raise ValueError("ResInfer MXFP4 supports dense Linear layers only")
            except ImportError:
                pass
            if not isinstance(layer, LinearBase):
                return None
            method = select_method(self, prefix, self.is_layer_excluded)
            return UnquantizedLinearMethod() if method is None else method
except Exception:                                           # no vLLM here: the method class above is all there is
    ModelOptMxfp4Config = None
