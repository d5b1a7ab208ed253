"""vLLM plugin: put the sm_100a kernels of this package under an unmodified vLLM.

Two hooks, both installed by ``register()`` (entry point of group ``vllm.general_plugins`` in the
pyproject.toml next to this package; vLLM loads those in the API server, the engine core and
every worker, vllm/plugins/__init__.py:28-82; the function is idempotent, as vLLM requires):

1. **Quantization configs.**  ``"awq"`` and ``"awq_marlin"`` are re-registered
   (vllm/model_executor/layers/quantization/__init__.py:59-106: a registered config replaces the
   built-in of the same name).  vLLM started without ``--quantization`` turns every AWQ
   checkpoint into ``awq_marlin`` (awq_marlin.py:249-278), so that name has to be covered for the
   kernels to be reached at all.  Both configs hand out
     * ``B200AWQLinearMethod`` for linear layers: vLLM's own ``create_weights`` (the checkpoint
       loaders keep working), no Marlin repack, ``apply`` = one fused kernel family for every
       token count (awq.py:262-286 switches to dequantize + matmul at 256 tokens);
     * ``B200AWQMoEMethod`` for fused-MoE layers: the AWQ-layout stacked parameters of
       awq_marlin.py:549-623 kept as they are, ``apply`` with the signature of
       fused_moe_method_base.py:163-172 calling the expert kernels of this package.
   Layers the kernels cannot take (group sizes other than 32/64/128 for experts, odd hidden
   sizes) fall back to what stock vLLM would have picked.
2. **Operator overrides.**  ``torch.ops._C.awq_gemm`` / ``awq_dequantize`` are re-implemented for
   the CUDA dispatch key with ``allow_override=True`` so that any remaining call site that uses
   the literal op names (vllm/_custom_ops.py:542-605) lands here too.

Options (keyword arguments of ``register`` or the environment variables in brackets, which is
what a vLLM that loads the plug-in itself sees):
  repack_decode  [AWQ_B200_REPACK_DECODE=1]  decode-layout copies of ``qweight`` for <= 8 tokens
  decode_kmajor  [AWQ_B200_DECODE_KMAJOR=1]  K-major copies of the largest layers for 9..16 tokens
  dummy_fill     [AWQ_B200_DUMMY_FILL=seed]  after loading, overwrite the integer parameters and
                 scales from a seeded generator: ``--load-format dummy`` leaves integer
                 parameters uninitialised (model_loader/weight_utils.py:1484-1490) and draws
                 float ones from +-1e-3, not the nibble-uniform / scale-uniform[0.002, 0.02]
                 distributions of the benchmark.
  mode           [AWQ_B200_MODE=kernels|fill_only]  fill_only leaves vLLM's own methods in place
                 and only applies the seeded fill before them (the stock column of a comparison)
``calls`` counts how often each method ran (for tests that must see these kernels, not vLLM's).
"""
from __future__ import annotations

import os
import zlib

import torch

from . import ops, torch_ops
from .linear import kmajor_pays

_registered = False
_lib_handle = None
_options = {"repack_decode": False, "decode_kmajor": False, "dummy_fill": None}
calls = {"linear": 0, "moe": 0, "awq_gemm_op": 0, "awq_dequantize_op": 0}


def _awq_gemm(input, qweight, scales, qzeros, split_k_iters):
    calls["awq_gemm_op"] += 1
    return ops.awq_gemm(input.contiguous(), qweight, scales, qzeros, int(split_k_iters))


def _awq_dequantize(qweight, scales, zeros, split_k_iters, thx, thy):
    calls["awq_dequantize_op"] += 1
    return ops.awq_dequantize(qweight, scales, zeros, int(split_k_iters), int(thx), int(thy))


def fill_awq_tensors(qweight, scales, qzeros, seed: int) -> None:
    """Seeded benchmark distributions, in place: nibbles uniform 0..15, scales uniform
    [0.002, 0.02].  Drawn on the parameters' device."""
    gen = torch.Generator(device=qweight.device).manual_seed(int(seed))
    for t in (qweight, qzeros):
        t.copy_(torch.randint(-(2 ** 31), 2 ** 31, t.shape, dtype=torch.int64, device=t.device,
                              generator=gen).to(torch.int32))
    scales.copy_((0.002 + 0.018 * torch.rand(scales.shape, device=scales.device, generator=gen))
                 .to(scales.dtype))


def _name_seed(layer) -> int:
    """A per-layer offset that is the same in every process (str hashes are salted)."""
    return zlib.crc32(str(getattr(layer, "prefix", getattr(layer, "layer_name", ""))).encode())


def _build_methods():
    """The vLLM-derived classes, built on first use (importing vLLM's layer modules is heavy and
    needs its compiled ops)."""
    from vllm.model_executor.layers.fused_moe import (FusedMoEMethodBase,
                                                      FusedMoeWeightScaleSupported, RoutedExperts)
    from vllm.model_executor.layers.linear import LinearBase, UnquantizedLinearMethod
    from vllm.model_executor.layers.quantization import register_quantization_config
    from vllm.model_executor.layers.quantization.awq import AWQConfig, AWQLinearMethod
    from vllm.model_executor.layers.quantization.awq_marlin import AWQMarlinConfig
    from vllm.model_executor.layers.quantization.utils.quant_utils import is_layer_skipped
    from vllm.model_executor.utils import set_weight_attrs

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

    register_quantization_config("awq")(B200AWQConfig)
    register_quantization_config("awq_marlin")(B200AWQMarlinConfig)
    return {"linear": B200AWQLinearMethod, "moe": B200AWQMoEMethod, "awq": B200AWQConfig,
            "awq_marlin": B200AWQMarlinConfig}


classes: dict = {}


def _install_fill_only() -> None:
    """Stock vLLM methods, same weights: the seeded fill runs before vLLM's own
    ``process_weights_after_loading`` (Marlin repack included), nothing else changes.  This is
    the stock column of the serving comparison."""
    from vllm.model_executor.layers.quantization.awq import AWQLinearMethod
    from vllm.model_executor.layers.quantization.awq_marlin import (AWQMarlinLinearMethod,
                                                                    AWQMarlinMoEMethod)

    def wrap_linear(cls):
        stock = cls.process_weights_after_loading

        def process(self, layer):
            if _options["dummy_fill"] is not None:
                fill_awq_tensors(layer.qweight.data, layer.scales.data, layer.qzeros.data,
                                 _options["dummy_fill"] + _name_seed(layer))
            return stock(self, layer)

        cls.process_weights_after_loading = process

    wrap_linear(AWQLinearMethod)
    wrap_linear(AWQMarlinLinearMethod)
    stock_moe = AWQMarlinMoEMethod.process_weights_after_loading

    def process_moe(self, layer):
        if _options["dummy_fill"] is not None:
            seed = _options["dummy_fill"] + _name_seed(layer)
            fill_awq_tensors(layer.w13_qweight.data, layer.w13_scales.data,
                             layer.w13_qzeros.data, seed + 1)
            fill_awq_tensors(layer.w2_qweight.data, layer.w2_scales.data,
                             layer.w2_qzeros.data, seed + 2)
        return stock_moe(self, layer)

    AWQMarlinMoEMethod.process_weights_after_loading = process_moe


def register(full_gemm: bool = True, repack_decode: bool = False, decode_kmajor: bool = False,
             dummy_fill: int | None = None, mode: str | None = None) -> None:
    """Install the hooks.  Needs vLLM's compiled ops to be importable (the op schemas are defined
    by vllm._C).  ``mode`` [AWQ_B200_MODE]: "kernels" (default: both hooks of the module text) or
    "fill_only" (stock vLLM kernels on the seeded weights).  ``full_gemm`` is kept for callers of
    the earlier signature: the linear method uses the fused kernels for every token count."""
    global _registered, _lib_handle
    env = os.environ.get
    _options["repack_decode"] = repack_decode or env("AWQ_B200_REPACK_DECODE") == "1"
    _options["decode_kmajor"] = decode_kmajor or env("AWQ_B200_DECODE_KMAJOR") == "1"
    if dummy_fill is None and env("AWQ_B200_DUMMY_FILL") not in (None, ""):
        dummy_fill = int(env("AWQ_B200_DUMMY_FILL"))
    _options["dummy_fill"] = dummy_fill
    if _registered:
        return
    mode = mode or env("AWQ_B200_MODE") or "kernels"
    if mode == "fill_only":
        _install_fill_only()
        _registered = True
        return
    if mode != "kernels":
        raise ValueError("mode is 'kernels' or 'fill_only'")
    import vllm._C  # noqa: F401  (defines the _C op schemas)
    lib = torch.library.Library("_C", "IMPL")
    lib.impl("awq_gemm", _awq_gemm, "CUDA", allow_override=True)
    lib.impl("awq_dequantize", _awq_dequantize, "CUDA", allow_override=True)
    _lib_handle = lib  # keep the registration alive
    classes.update(_build_methods())
    _registered = True
