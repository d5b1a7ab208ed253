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

import ctypes

import torch
import torch.distributed as dist

from . import _lib, ops

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
                         group=None, comm: "PeerAllReduce | None" = None,
                         slot: int = 0) -> torch.Tensor:
    """y [M, N] = sum over ranks of x_shard @ W_shard; the bias is added on rank 0 only so that
    the sum holds it once.  With ``comm`` the GEMM writes its partial straight into this rank's
    peer-mapped region and the one-shot kernel sums the regions (consecutive calls alternate
    ``slot`` 0 / 1); without it the partial is all-reduced by NCCL."""
    qweight, scales, qzeros = shard
    rank0 = (not dist.is_initialized()) or dist.get_rank(group) == 0
    b = bias if rank0 else None
    if comm is not None and comm.fits(x_shard.shape[0], scales.shape[1]):
        partial = comm.partial(slot, x_shard.shape[0], scales.shape[1])
        ops.awq_gemm(x_shard, qweight, scales, qzeros, PACK_FACTOR, bias=b, out=partial)
        return comm.reduce(slot, x_shard.shape[0], scales.shape[1])
    y = ops.awq_gemm(x_shard, qweight, scales, qzeros, PACK_FACTOR, bias=b)
    return all_reduce_output(y, group)


FLAG_BYTES = 4096      # AWQ_B200_AR_FLAG_BYTES
MAX_RANKS = 8          # AWQ_B200_AR_MAX_RANKS


def region_layout(max_bytes: int) -> tuple[int, int, int]:
    """(offset of slot 0, offset of slot 1, region size) for partials of up to ``max_bytes``."""
    per = -(-max_bytes // 256) * 256
    return FLAG_BYTES, FLAG_BYTES + per, FLAG_BYTES + 2 * per


def slot_for_call(call_index: int) -> int:
    """Consecutive all-reduce calls alternate between the two slots: a rank cannot enter call
    i + 2 before every peer has left call i, so a slot is never overwritten while it is read."""
    return call_index & 1


class PeerAllReduce:
    """Peer-mapped regions of the ranks of one node and the one-shot all-reduce over them
    (``awq_b200_allreduce``).  Set-up is collective over ``group``: every rank allocates its
    region, the CUDA IPC handles travel through torch.distributed, every rank maps the others'
    regions and enables peer access.  No multicast object is involved."""

    def __init__(self, max_bytes: int, group=None, device: torch.device | None = None) -> None:
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.off0, self.off1, size = region_layout(max_bytes)
        self.max_bytes = max_bytes
        # a dedicated allocation (not a slice of the caching allocator's pool would be shared as a
        # whole block; the offset inside the block travels with the handle)
        self.region = torch.zeros(size, dtype=torch.uint8, device=self.device)
        torch.cuda.synchronize(self.device)
        info = self.region.untyped_storage()._share_cuda_()
        infos = [None] * self.world
        dist.all_gather_object(infos, info, group=group)
        lib = _lib.load()
        self._peers = []        # keeps the mapped storages alive
        ptrs = []
        for r in range(self.world):
            if r == self.rank:
                ptrs.append(self.region.data_ptr())
                continue
            _lib.check("awq_b200_enable_peer_access",
                       lib.awq_b200_enable_peer_access(int(infos[r][0])))
            storage = torch.UntypedStorage._new_shared_cuda(*infos[r])
            self._peers.append(storage)
            ptrs.append(storage.data_ptr())
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self.state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.calls = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)   # every region is zeroed and mapped before the first call

    def fits(self, m: int, n: int) -> bool:
        return 0 < m * n * 2 <= self.max_bytes and (m * n * 2) % 16 == 0

    def partial(self, slot: int, m: int, n: int) -> torch.Tensor:
        """This rank's fp16 [m, n] partial inside its region (what the GEMM writes)."""
        off = self.off1 if slot else self.off0
        return self.region[off:off + m * n * 2].view(torch.float16).view(m, n)

    def reduce(self, slot: int, m: int, n: int, out: torch.Tensor | None = None,
               end_barrier: bool = False, dependent_launch: bool = True) -> torch.Tensor:
        if out is None:
            out = torch.empty((m, n), dtype=torch.float16, device=self.device)
        flags = int(end_barrier) | (2 if dependent_launch else 0)
        rc = _lib.load().awq_b200_allreduce(
            self._ptrs, self.rank, self.world, self.off1 if slot else self.off0, out.data_ptr(),
            m * n * 2, self.state.data_ptr(), flags, torch.cuda.current_stream().cuda_stream)
        _lib.check("awq_b200_allreduce", rc)
        self.calls += 1
        return out

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum of the ranks' ``partial`` tensors (copied into the region first; the fused path,
        where the GEMM writes the region itself, is ``row_parallel_forward(..., comm=)``)."""
        m, n = partial.shape
        slot = slot_for_call(self.calls)
        self.partial(slot, m, n).copy_(partial)
        return self.reduce(slot, m, n, dependent_launch=False)
