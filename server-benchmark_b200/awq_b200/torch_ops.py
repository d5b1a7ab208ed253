"""The linear op as a registered torch operator, ``torch.ops.awq_b200.linear``.

vLLM traces ``quant_method.apply`` of linear layers with torch.compile (``fullgraph=True``) and
captures the result in CUDA graphs; a ctypes call is not traceable, a registered operator with a
fake implementation is (vLLM's own ops do the same, vllm/_custom_ops.py:559-605).  The token count
is symbolic while tracing, so the choice between the weight layouts (decode-layout copy for
<= 8 tokens, K-major copy for 9..16, checkpoint layout above) is made inside the operator, at run
time, where the count is a number.
"""
from __future__ import annotations

import torch

from . import _lib, ops
from .linear import KMAJOR_TOKENS, REPACK_MAX_TOKENS

_fragment = torch.library.Library("awq_b200", "FRAGMENT")
_fragment.define("linear(Tensor x, Tensor qweight, Tensor scales, Tensor qzeros, Tensor? bias, "
                 "Tensor? qweight_decode, Tensor? qweight_kmajor) -> Tensor")


def _linear(x, qweight, scales, qzeros, bias, qweight_decode, qweight_kmajor):
    tokens = x.shape[0]
    if qweight_decode is not None and tokens <= REPACK_MAX_TOKENS:
        return ops.awq_gemm(x, qweight_decode, scales, qzeros, 8, bias=bias,
                            kernel=_lib.KERNEL_STREAM_RP)
    if qweight_kmajor is not None and KMAJOR_TOKENS[0] <= tokens <= KMAJOR_TOKENS[1]:
        return ops.awq_gemm(x, qweight_kmajor, scales, qzeros, 8, bias=bias,
                            kernel=_lib.KERNEL_Q8)
    return ops.awq_gemm(x, qweight, scales, qzeros, 8, bias=bias)


def _linear_fake(x, qweight, scales, qzeros, bias, qweight_decode, qweight_kmajor):
    return x.new_empty((x.shape[0], scales.shape[1]))


_fragment.impl("linear", _linear, "CUDA")
torch.library.register_fake("awq_b200::linear", _linear_fake, lib=_fragment)

linear = torch.ops.awq_b200.linear
