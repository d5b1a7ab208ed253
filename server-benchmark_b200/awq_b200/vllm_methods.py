"""The vLLM-derived classes of the plug-in, at module level so that vLLM can pickle a config that
holds them by reference when it spawns its engine processes (classes made inside a function are
pickled by value, together with everything their methods name).  Importing this module imports
vLLM's layer modules; ``awq_b200.vllm_plugin.register`` does so on first use."""
from __future__ import annotations

import torch
from vllm.model_executor.layers.fused_moe import (FusedMoEMethodBase,
                                                  FusedMoeWeightScaleSupported, RoutedExperts)
from vllm.model_executor.layers.linear import LinearBase, UnquantizedLinearMethod
from vllm.model_executor.layers.quantization.awq import AWQConfig, AWQLinearMethod
from vllm.model_executor.layers.quantization.awq_marlin import AWQMarlinConfig
from vllm.model_executor.layers.quantization.moe_wna16 import (MoeWNA16Config, MoeWNA16Method,
                                                                 is_layer_skipped_quant)
from vllm.model_executor.layers.quantization.utils.quant_utils import is_layer_skipped
from vllm.model_executor.utils import set_weight_attrs

from . import ops, torch_ops
from .linear import kmajor_pays
from .vllm_plugin import _name_seed, _options, calls, fill_awq_tensors


class B200AWQLinearMethod(AWQLinearMethod):
    """AWQLinearMethod (awq.py:172-286) with the parameter contract unchanged and ``apply``
    on this package's kernels."""

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        for name in ("qweight", "qzeros", "scales"):
            p = getattr(layer, name)
            setattr(layer, name, torch.nn.Parameter(p.data.contiguous(), requires_grad=False))
        if _options["dummy_fill"] is not None:
            fill_awq_tensors(layer.qweight.data, layer.scales.data, layer.qzeros.data,
                             _options["dummy_fill"] + _name_seed(layer))
        k, words = layer.qweight.shape
        group = k // layer.scales.shape[0]
        layer.qweight_decode = None
        layer.qweight_kmajor = None
        if _options["repack_decode"] and group == 128 and k % 128 == 0 and words % 4 == 0:
            layer.qweight_decode = ops.awq_repack(layer.qweight.data)
        if _options["decode_kmajor"] and kmajor_pays(layer.qweight.data, group):
            layer.qweight_kmajor = ops.awq_repack_kmajor(layer.qweight.data)

    def apply(self, layer, x, bias=None):
        # traced by torch.compile inside vLLM: one registered operator, layout choice inside
        calls["linear"] += 1
        if x.dtype != torch.float16:
            raise ValueError("AWQ on B200 computes in fp16: start vLLM with --dtype half")
        out_shape = x.shape[:-1] + (layer.scales.shape[-1],)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        out = torch_ops.linear(x2, layer.qweight, layer.scales, layer.qzeros, bias,
                               getattr(layer, "qweight_decode", None),
                               getattr(layer, "qweight_kmajor", None))
        return out.reshape(out_shape)


class B200AWQMoEMethod(FusedMoEMethodBase):
    """Fused-MoE method on the AWQ checkpoint layout (parameters as
    awq_marlin.py:549-623 registers them, no Marlin or wna16 repack)."""

    def __init__(self, quant_config, moe):
        super().__init__(moe)
        self.quant_config = quant_config

    def create_weights(self, layer, num_experts: int, hidden_size: int,
                       intermediate_size_per_partition: int, params_dtype: torch.dtype,
                       **extra_weight_attrs):
        extra_weight_attrs.update({"is_transposed": True,
                                   "quant_method": FusedMoeWeightScaleSupported.GROUP.value})
        extra_weight_attrs.pop("intermediate_size_full", None)
        pf = self.quant_config.pack_factor
        g = self.quant_config.group_size
        inter = intermediate_size_per_partition

        def add(name, shape, dtype):
            p = torch.nn.Parameter(torch.empty(*shape, dtype=dtype), requires_grad=False)
            layer.register_parameter(name, p)
            set_weight_attrs(p, extra_weight_attrs)

        add("w13_qweight", (num_experts, hidden_size, 2 * inter // pf), torch.int32)
        add("w2_qweight", (num_experts, inter, hidden_size // pf), torch.int32)
        add("w13_scales", (num_experts, hidden_size // g, 2 * inter), params_dtype)
        add("w2_scales", (num_experts, inter // g, hidden_size), params_dtype)
        add("w13_qzeros", (num_experts, hidden_size // g, 2 * inter // pf), torch.int32)
        add("w2_qzeros", (num_experts, inter // g, hidden_size // pf), torch.int32)
        layer.num_groups_w13 = hidden_size // g
        layer.num_groups_w2 = inter // g

    def process_weights_after_loading(self, layer) -> None:
        for name in ("w13_qweight", "w2_qweight", "w13_scales", "w2_scales", "w13_qzeros",
                     "w2_qzeros"):
            p = getattr(layer, name)
            setattr(layer, name, torch.nn.Parameter(p.data.contiguous(), requires_grad=False))
        if _options["dummy_fill"] is not None:
            seed = _options["dummy_fill"] + _name_seed(layer)
            fill_awq_tensors(layer.w13_qweight.data, layer.w13_scales.data,
                             layer.w13_qzeros.data, seed + 1)
            fill_awq_tensors(layer.w2_qweight.data, layer.w2_scales.data,
                             layer.w2_qzeros.data, seed + 2)
        self.moe_quant_config = None   # rebuilt from the final parameters on first use
        layer.w13_decode = layer.w2_decode = None
        if _options["repack_decode"] and self.quant_config.group_size == 128:
            layer.w13_decode = ops.awq_repack(layer.w13_qweight.data)
            layer.w2_decode = ops.awq_repack(layer.w2_qweight.data)

    def get_fused_moe_quant_config(self, layer):
        # built after loading (layer.ensure_moe_quant_config_init): scales and zero points
        # ride in vLLM's own container, as for the Marlin method (awq_marlin.py:708-731)
        from vllm.model_executor.layers.fused_moe.config import awq_marlin_moe_quant_config
        return awq_marlin_moe_quant_config(
            w1_scale=layer.w13_scales, w2_scale=layer.w2_scales,
            w1_zp=layer.w13_qzeros, w2_zp=layer.w2_qzeros,
            weight_bits=self.quant_config.weight_bits,
            group_size=self.quant_config.group_size)

    def apply(self, layer, x, topk_weights, topk_ids, shared_experts=None,
              shared_experts_input=None):
        calls["moe"] += 1
        if x.dtype != torch.float16:
            raise ValueError("AWQ on B200 computes in fp16: start vLLM with --dtype half")
        if self.moe_quant_config is None:
            self.moe_quant_config = self.get_fused_moe_quant_config(layer)
        act = getattr(layer, "activation", "silu")
        return ops.fused_experts(
            x.contiguous(), layer.w13_qweight, layer.w2_qweight,
            topk_weights.to(torch.float32).contiguous(),
            topk_ids.to(torch.int32).contiguous(),
            activation=str(getattr(act, "value", act)),
            apply_router_weight_on_input=getattr(layer, "apply_router_weight_on_input", False),
            global_num_experts=getattr(layer, "global_num_experts", -1),
            expert_map=getattr(layer, "expert_map", None),
            w1_decode=getattr(layer, "w13_decode", None),
            w2_decode=getattr(layer, "w2_decode", None),
            quant_config=self.moe_quant_config)


def moe_supported(layer, group_size: int) -> bool:
    h = getattr(layer, "hidden_size", None)
    inter = getattr(layer, "intermediate_size_per_partition", None)
    if h is None or inter is None:
        return True
    return group_size in (32, 64, 128) and h % 128 == 0 and inter % 128 == 0


def quant_method_for(cfg, stock_cls, layer, prefix):
    if isinstance(layer, LinearBase):
        if is_layer_skipped(prefix, cfg.modules_to_not_convert,
                            getattr(cfg, "packed_modules_mapping", {}), skip_with_substr=True):
            return UnquantizedLinearMethod()
        return B200AWQLinearMethod(cfg)
    if isinstance(layer, RoutedExperts):
        if moe_supported(layer, cfg.group_size):
            return B200AWQMoEMethod(cfg, layer.moe_config)
    return stock_cls.get_quant_method(cfg, layer, prefix)


class B200AWQConfig(AWQConfig):
    """``awq`` (awq.py:36-170) handing out the B200 methods."""

    def get_quant_method(self, layer, prefix):
        return quant_method_for(self, AWQConfig, layer, prefix)


class B200AWQMarlinConfig(AWQMarlinConfig):
    """``awq_marlin`` (awq_marlin.py:168-345), the name every AWQ checkpoint is overridden
    to when vLLM is started without --quantization, handing out the B200 methods."""

    def get_quant_method(self, layer, prefix):
        return quant_method_for(self, AWQMarlinConfig, layer, prefix)


class B200MoeWNA16Method(MoeWNA16Method):
    """MoeWNA16Method (moe_wna16.py:208-512) with its parameter declaration and checkpoint
    loader unchanged -- the loader converts AWQ expert tensors to uint8 [E, N, K/2] while it
    loads -- and, once loading is over, the tensors converted back to the AWQ layout the expert
    kernels read (one pass at load time, ``ops.wna16_to_awq``)."""

    def process_weights_after_loading(self, layer) -> None:
        g = layer.group_size
        if _options["dummy_fill"] is not None:
            gen = torch.Generator(device=layer.w13_qweight.device).manual_seed(
                _options["dummy_fill"] + _name_seed(layer))
            for name in ("w13_qweight", "w2_qweight", "w13_qzeros", "w2_qzeros"):
                p = getattr(layer, name)
                p.data.copy_(torch.randint(0, 256, p.shape, dtype=torch.int32, device=p.device,
                                           generator=gen).to(torch.uint8))
            for name in ("w13_scales", "w2_scales"):
                p = getattr(layer, name)
                p.data.copy_((0.002 + 0.018 * torch.rand(p.shape, device=p.device,
                                                         generator=gen)).to(p.dtype))
        for proj in ("w13", "w2"):
            q, s, z = ops.wna16_to_awq(getattr(layer, proj + "_qweight").data.contiguous(),
                                       getattr(layer, proj + "_scales").data.contiguous(),
                                       getattr(layer, proj + "_qzeros").data.contiguous(), g)
            for name, t in (("_qweight", q), ("_scales", s), ("_qzeros", z)):
                setattr(layer, proj + name, torch.nn.Parameter(t, requires_grad=False))
        self.moe_quant_config = None

    def get_fused_moe_quant_config(self, layer):
        from vllm.model_executor.layers.fused_moe.config import int4_w4a16_moe_quant_config
        return int4_w4a16_moe_quant_config(
            w1_scale=layer.w13_scales, w2_scale=layer.w2_scales, w1_zp=layer.w13_qzeros,
            w2_zp=layer.w2_qzeros, block_shape=[0, layer.group_size])

    def apply(self, layer, x, topk_weights, topk_ids, shared_experts=None,
              shared_experts_input=None):
        calls["moe"] += 1
        if x.dtype != torch.float16:
            raise ValueError("AWQ on B200 computes in fp16: start vLLM with --dtype half")
        if self.moe_quant_config is None:
            self.moe_quant_config = self.get_fused_moe_quant_config(layer)
        act = getattr(layer, "activation", "silu")
        return ops.fused_experts(
            x.contiguous(), layer.w13_qweight, layer.w2_qweight,
            topk_weights.to(torch.float32).contiguous(), topk_ids.to(torch.int32).contiguous(),
            activation=str(getattr(act, "value", act)),
            apply_router_weight_on_input=getattr(layer, "apply_router_weight_on_input", False),
            global_num_experts=getattr(layer, "global_num_experts", -1),
            expert_map=getattr(layer, "expert_map", None), quant_config=self.moe_quant_config)


class B200MoeWNA16Config(MoeWNA16Config):
    """``moe_wna16`` (moe_wna16.py:34-206) handing out the B200 methods for AWQ checkpoints;
    GPTQ checkpoints and shapes the expert kernels do not take stay on vLLM's own methods."""

    def get_quant_method(self, layer, prefix):
        awq = self.linear_quant_method in ("awq", "awq_marlin") and self.weight_bits == 4 \
            and self.has_zp
        if not awq or is_layer_skipped_quant(prefix, self.modules_to_not_convert):
            return MoeWNA16Config.get_quant_method(self, layer, prefix)
        if isinstance(layer, LinearBase):
            return B200AWQConfig.from_config(self.full_config).get_quant_method(layer, prefix)
        if isinstance(layer, RoutedExperts) and moe_supported(layer, self.group_size):
            return B200MoeWNA16Method(self, layer.moe_config)
        return MoeWNA16Config.get_quant_method(self, layer, prefix)
