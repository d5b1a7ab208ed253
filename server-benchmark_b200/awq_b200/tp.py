"""Tensor-parallel AWQ linears: one process per GPU, torch.distributed (NCCL over NVLink) for the
exchange step.

Mirrors vLLM's parallel linear layers for AWQ weights (paths inside the ``vllm`` package):
  column-parallel (qkv, gate_up): split N, no collective      model_executor/layers/linear.py:578-596
  row-parallel (o_proj, down):    split K, all-reduce of the fp16 [M, hidden] partial outputs,
                                  bias on rank 0 only          model_executor/layers/linear.py:1540-1566
                                                               distributed/communication_op.py:12-14
Shards keep the AWQ layout, so the same kernels run on every rank.  K is split on group
boundaries (K_part % group_size == 0 is what create_weights demands, quantization/awq.py:198-203);
a K whose group count does not divide by the TP degree is first padded with zero-contribution
groups (``pad_k_for_tp``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops

PACK_FACTOR = 8


def shard_columns(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
                  rank: int, world: int):
    """Column-parallel shard: output columns [rank * N/world, (rank + 1) * N/world)."""
    n = scales.shape[1]
    if n % (world * PACK_FACTOR) != 0:
        raise ValueError("The output size is not aligned with the quantized weight shape. "
                         "This can be caused by too large tensor parallel size.")
    per = n // world
    w0, w1 = rank * per // PACK_FACTOR, (rank + 1) * per // PACK_FACTOR
    return (qweight[:, w0:w1].contiguous(), scales[:, rank * per:(rank + 1) * per].contiguous(),
            qzeros[:, w0:w1].contiguous())


def shard_rows(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
               rank: int, world: int):
    """Row-parallel shard: input rows [rank * K/world, (rank + 1) * K/world), whole groups only."""
    k = qweight.shape[0]
    groups = scales.shape[0]
    group = k // groups
    if groups % world != 0:
        raise ValueError("The input size is not aligned with the quantized weight shape. "
                         "This can be caused by too large tensor parallel size.")
    gper = groups // world
    g0, g1 = rank * gper, (rank + 1) * gper
    return (qweight[g0 * group:g1 * group].contiguous(), scales[g0:g1].contiguous(),
            qzeros[g0:g1].contiguous())


def pad_k_for_tp(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor, world: int):
    """Append whole groups whose weights dequantise to zero (q = z = 0) until the group count
    divides by ``world``.  The matching activation columns must be zero-padded too
    (``pad_x_for_tp``); the product is unchanged."""
    k = qweight.shape[0]
    groups = scales.shape[0]
    group = k // groups
    extra = (-groups) % world
    if extra == 0:
        return qweight, scales, qzeros
    qweight = torch.cat([qweight, qweight.new_zeros(extra * group, qweight.shape[1])])
    scales = torch.cat([scales, scales.new_zeros(extra, scales.shape[1])])
    qzeros = torch.cat([qzeros, qzeros.new_zeros(extra, qzeros.shape[1])])
    return qweight, scales, qzeros


def pad_x_for_tp(x: torch.Tensor, k_padded: int) -> torch.Tensor:
    if x.shape[-1] == k_padded:
        return x
    return torch.nn.functional.pad(x, (0, k_padded - x.shape[-1]))


def shard_input(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The slice of the activations a row-parallel rank multiplies (input_is_parallel)."""
    k = x.shape[-1]
    per = k // world
    return x[..., rank * per:(rank + 1) * per].contiguous()


def all_reduce_output(partial: torch.Tensor, group=None) -> torch.Tensor:
    """tensor_model_parallel_all_reduce: sum of the ranks' partial outputs, in place."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def column_parallel_forward(x: torch.Tensor, shard, bias_shard: torch.Tensor | None = None):
    """y_shard [M, N/world]; outputs stay sharded (gather_output=False)."""
    qweight, scales, qzeros = shard
    return ops.awq_gemm(x, qweight, scales, qzeros, PACK_FACTOR, bias=bias_shard)


def row_parallel_forward(x_shard: torch.Tensor, shard, bias: torch.Tensor | None = None,
                         group=None) -> torch.Tensor:
    """y [M, N] = sum over ranks of x_shard @ W_shard; the bias is added on rank 0 only so that
    the sum holds it once."""
    qweight, scales, qzeros = shard
    rank0 = (not dist.is_initialized()) or dist.get_rank(group) == 0
    y = ops.awq_gemm(x_shard, qweight, scales, qzeros, PACK_FACTOR, bias=bias if rank0 else None)
    return all_reduce_output(y, group)
