"""vLLM plugin: route vLLM's AWQ ops to the sm_100a kernels of this package.

vLLM's AWQ linear method calls ``torch.ops._C.awq_gemm`` (fewer than 256 tokens) or
``torch.ops._C.awq_dequantize`` + ``torch.matmul`` (vllm/model_executor/layers/quantization/awq.py:
262-286, vllm/_custom_ops.py:542-587).  ``register()`` re-implements both ops for the CUDA
dispatch key with ``allow_override=True``, so every call site keeps its literal op name and the
model code, CUDA-graph capture and torch.compile tracing of vLLM are untouched.

It is exposed as an entry point of group ``vllm.general_plugins`` (see pyproject.toml next to
this package; vLLM loads those in the API server, the engine core and every worker:
vllm/plugins/__init__.py:28-82).  The function is idempotent, as vLLM requires.

``register(full_gemm=True)`` additionally makes AWQLinearMethod.apply call the fused kernel for
every token count instead of materialising the fp16 weight matrix for >= 256 tokens.
``register(repack_decode=True)`` (implies full_gemm) also makes
AWQLinearMethod.process_weights_after_loading keep a decode-layout copy of every ``qweight``
(ops.awq_repack: a second copy of the int4 weights) which ``apply`` uses for up to 8 tokens.
When vLLM loads the plug-in itself it calls ``register()`` without arguments; the environment
variables AWQ_B200_FULL_GEMM=1 and AWQ_B200_REPACK_DECODE=1 select the options then.
"""
from __future__ import annotations

import os

import torch

from . import _lib, ops

_registered = False
_lib_handle = None


def _awq_gemm(input, qweight, scales, qzeros, split_k_iters):
    return ops.awq_gemm(input.contiguous(), qweight, scales, qzeros, int(split_k_iters))


def _awq_dequantize(qweight, scales, zeros, split_k_iters, thx, thy):
    return ops.awq_dequantize(qweight, scales, zeros, int(split_k_iters), int(thx), int(thy))


def register(full_gemm: bool = False, repack_decode: bool = False) -> None:
    """Override torch.ops._C.awq_gemm / awq_dequantize on CUDA.  Needs vLLM's compiled ops to be
    importable (the op schemas are defined by vllm._C)."""
    global _registered, _lib_handle
    full_gemm = full_gemm or os.environ.get("AWQ_B200_FULL_GEMM") == "1"
    repack_decode = repack_decode or os.environ.get("AWQ_B200_REPACK_DECODE") == "1"
    full_gemm = full_gemm or repack_decode
    if not _registered:
        import vllm._C  # noqa: F401  (defines the _C op schemas)
        lib = torch.library.Library("_C", "IMPL")
        lib.impl("awq_gemm", _awq_gemm, "CUDA", allow_override=True)
        lib.impl("awq_dequantize", _awq_dequantize, "CUDA", allow_override=True)
        _lib_handle = lib  # keep the registration alive
        _registered = True
    if full_gemm:
        from vllm.model_executor.layers.quantization import awq as vllm_awq

        def apply(self, layer, x, bias=None):
            qweight, scales, qzeros = layer.qweight, layer.scales, layer.qzeros
            out_shape = x.shape[:-1] + (qweight.shape[-1] * self.quant_config.pack_factor,)
            x2 = x.reshape(-1, x.shape[-1]).contiguous()
            decode = getattr(layer, "qweight_decode", None)
            if decode is not None and x2.shape[0] <= 8:
                out = ops.awq_gemm(x2, decode, scales, qzeros, self.quant_config.pack_factor,
                                   bias=bias, kernel=_lib.KERNEL_STREAM_RP)
            else:
                out = ops.awq_gemm(x2, qweight, scales, qzeros, self.quant_config.pack_factor,
                                   bias=bias)
            return out.reshape(out_shape)

        vllm_awq.AWQLinearMethod.apply = apply
    if repack_decode:
        from vllm.model_executor.layers.quantization import awq as vllm_awq

        if not getattr(vllm_awq.AWQLinearMethod, "_awq_b200_repack", False):
            original = vllm_awq.AWQLinearMethod.process_weights_after_loading

            def process_weights_after_loading(self, layer):
                original(self, layer)
                k, words = layer.qweight.shape
                group = k // layer.scales.shape[0]
                layer.qweight_decode = None
                if group == 128 and k % 128 == 0 and words % 4 == 0:
                    layer.qweight_decode = ops.awq_repack(layer.qweight.data.contiguous())

            vllm_awq.AWQLinearMethod.process_weights_after_loading = process_weights_after_loading
            vllm_awq.AWQLinearMethod._awq_b200_repack = True
