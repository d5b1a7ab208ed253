"""awq_b200 -- B200-native (sm_100a) AWQ W4A16 linear and fused-MoE kernels behind the
operator API of the vLLM ops the cloudrift-ai/server-benchmark harness measures.

Host code is Python; all arithmetic runs in libawq_b200.so (hand-written CUDA, C ABI in
include/awq_b200.h).  There is no CPU or eager fallback: importing the ops without the built
library raises.
"""
from . import _lib  # noqa: F401
from ._lib import (KERNEL_AUTO, KERNEL_GENERIC, KERNEL_STREAM, KERNEL_STREAM_EXACT,  # noqa: F401
                   KERNEL_TCGEN05, KERNEL_TS, KERNEL_TS_EXACT, KERNEL_WT, KERNEL_STREAM_RP, KERNEL_Q8,
                   AwqB200Error)
from .ops import (awq_dequantize, awq_gemm, awq_repack, awq_repack_kmajor, fused_experts, fused_moe, fused_topk,  # noqa: F401
                  moe_align_block_size, moe_workspace_bytes, reserve_workspace, wna16_to_awq)
from .linear import AWQConfig, AWQLinearMethod, AWQLinear  # noqa: F401

__version__ = "0.1"
