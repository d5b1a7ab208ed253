"""Layer-level API mirroring vLLM's AWQ linear method (paths inside the ``vllm`` package):

  AWQConfig            model_executor/layers/quantization/awq.py:36-107
  AWQLinearMethod      model_executor/layers/quantization/awq.py:172-286
      create_weights   :182-255   parameter contract (qweight / qzeros / scales shapes, checks)
      apply            :262-286   y = x @ dequant(W) (+ bias), output shape x.shape[:-1] + (N,)

Difference from the reference: ``apply`` never materialises the fp16 weight matrix; one fused
kernel family serves every token count (the reference switches to dequantize + matmul at 256
tokens, awq.py:276-281).  ``AWQConfig(repack_decode=True)`` additionally keeps a decode-layout
copy of ``qweight`` (ops.awq_repack) that the streaming kernel reads for up to
``REPACK_MAX_TOKENS`` tokens; it costs a second copy of the int4 weights and is off by default.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib, ops

REPACK_MAX_TOKENS = 8  # the decode-layout kernel serves token counts up to this
KMAJOR_TOKENS = (9, 16)        # token counts the K-major kernel serves (measured: below, the
                               # streaming kernel on the decode layout is as fast or faster)
KMAJOR_MIN_TILES_PER_SM = 64   # layer size from which the K-major kernel wins (measured on the
                               # Qwen2.5-72B shapes: gate_up 100 tiles per SM 64 vs 83 us, down 50
                               # tiles per SM 43 vs 40 us)


@dataclass
class AWQConfig:
    """weight_bits is fixed at 4; pack_factor = 32 / weight_bits = 8 (awq.py:50-63)."""

    weight_bits: int = 4
    group_size: int = 128
    zero_point: bool = True
    repack_decode: bool = False
    decode_kmajor: bool = False

    def __post_init__(self) -> None:
        if self.weight_bits != 4:
            raise ValueError("Currently, only 4-bit weight quantization is supported for AWQ, "
                             f"but got {self.weight_bits} bits.")
        if not self.zero_point:
            raise ValueError("AWQ checkpoints without zero points are not supported")
        self.pack_factor = 32 // self.weight_bits

    @staticmethod
    def get_supported_act_dtypes() -> list[torch.dtype]:
        return [torch.half]

    @staticmethod
    def get_min_capability() -> int:
        return 100  # sm_100a only


def kmajor_pays(qweight: torch.Tensor, group_size: int) -> bool:
    """Whether the K-major decode kernel is the faster one for a layer of this size."""
    k, words = qweight.shape
    if group_size != 128 or k % 128 != 0 or k // 128 > 256:
        return False
    sms = torch.cuda.get_device_properties(qweight.device).multi_processor_count
    tiles = -(-words * 8 // 256) * (k // 128)
    return tiles >= KMAJOR_MIN_TILES_PER_SM * sms


class AWQLinear(torch.nn.Module):
    """Bare parameter holder, the role LinearBase plays for quant_method.create_weights."""

    def __init__(self) -> None:
        super().__init__()


class AWQLinearMethod:
    """Linear method for AWQ on B200."""

    def __init__(self, quant_config: AWQConfig):
        self.quant_config = quant_config

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, device: torch.device | str = "cuda",
                       **extra_weight_attrs) -> None:
        group_size = self.quant_config.group_size
        if group_size == -1:
            group_size = input_size
        if input_size_per_partition % group_size != 0:
            raise ValueError(
                "The input size is not aligned with the quantized weight shape. This can be "
                "caused by too large tensor parallel size.")
        output_size_per_partition = sum(output_partition_sizes)
        if output_size_per_partition % self.quant_config.pack_factor != 0:
            raise ValueError(
                "The output size is not aligned with the quantized weight shape. This can be "
                "caused by too large tensor parallel size.")
        if params_dtype != torch.float16:
            raise ValueError("AWQ supports fp16 activations only")
        pf = self.quant_config.pack_factor
        mk = lambda *shape, dtype: torch.nn.Parameter(  # noqa: E731
            torch.empty(*shape, dtype=dtype, device=device), requires_grad=False)
        layer.register_parameter(
            "qweight", mk(input_size_per_partition, output_size_per_partition // pf,
                          dtype=torch.int32))
        layer.register_parameter(
            "qzeros", mk(input_size_per_partition // group_size, output_size_per_partition // pf,
                         dtype=torch.int32))
        layer.register_parameter(
            "scales", mk(input_size_per_partition // group_size, output_size_per_partition,
                         dtype=params_dtype))
        layer.group_size = group_size

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        for name in ("qweight", "qzeros", "scales"):
            p = getattr(layer, name)
            setattr(layer, name, torch.nn.Parameter(p.data.contiguous(), requires_grad=False))
        layer.qweight_decode = None
        layer.qweight_kmajor = None
        k, words = layer.qweight.shape
        if (self.quant_config.repack_decode and layer.group_size == 128 and k % 128 == 0
                and words % 4 == 0):
            layer.qweight_decode = ops.awq_repack(layer.qweight.data)
        if self.quant_config.decode_kmajor and kmajor_pays(layer.qweight, layer.group_size):
            layer.qweight_kmajor = ops.awq_repack_kmajor(layer.qweight.data)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor,
              bias: torch.Tensor | None = None) -> torch.Tensor:
        qweight, scales, qzeros = layer.qweight, layer.scales, layer.qzeros
        pack_factor = self.quant_config.pack_factor
        out_shape = x.shape[:-1] + (qweight.shape[-1] * pack_factor,)
        reshaped_x = x.reshape(-1, x.shape[-1])
        if not reshaped_x.is_contiguous():
            reshaped_x = reshaped_x.contiguous()
        decode = getattr(layer, "qweight_decode", None)
        kmajor = getattr(layer, "qweight_kmajor", None)
        tokens = reshaped_x.shape[0]
        if decode is not None and tokens <= REPACK_MAX_TOKENS:
            out = ops.awq_gemm(reshaped_x, decode, scales, qzeros, pack_factor, bias=bias,
                               kernel=_lib.KERNEL_STREAM_RP)
        elif kmajor is not None and KMAJOR_TOKENS[0] <= tokens <= KMAJOR_TOKENS[1]:
            out = ops.awq_gemm(reshaped_x, kmajor, scales, qzeros, pack_factor, bias=bias,
                               kernel=_lib.KERNEL_Q8)
        else:
            out = ops.awq_gemm(reshaped_x, qweight, scales, qzeros, pack_factor, bias=bias)
        return out.reshape(out_shape)
