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


class _DeviceBytes:
    """Raw device memory as an object torch can alias (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


class PeerAllReduce:
    """Peer-mapped regions of the ranks of one node and the one-shot all-reduce over them
    (``awq_b200_allreduce``).  Set-up is collective over ``group``: every rank creates its region
    (``awq_b200_peer_region_create``), the CUDA IPC handles travel through torch.distributed, every
    rank maps the others' regions into its own device's context (``awq_b200_peer_region_open``).
    No multicast object is involved."""

    def __init__(self, max_bytes: int, group=None, device: torch.device | None = None) -> None:
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.off0, self.off1, size = region_layout(max_bytes)
        self.max_bytes = max_bytes
        lib = _lib.load()
        self._lib = lib
        self._opened: list[int] = []
        self._base = None
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)      # AWQ_B200_IPC_HANDLE_BYTES
            # a failure on one rank must not leave the others alone in a collective: every rank
            # goes through the same sequence (gather, agreement, barrier) whatever happens to it
            rc = lib.awq_b200_peer_region_create(size, ctypes.byref(base), handle)
            failure = None if rc == 0 else f"rank {self.rank} could not create its region (code {rc})"
            self._base = base.value if rc == 0 else None
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw if rc == 0 else None, group=group)
            if failure is None and any(h is None for h in handles):
                failure = "another rank could not create its region"
            ptrs = []
            for r in range(self.world):
                if failure is not None:
                    break
                if r == self.rank:
                    ptrs.append(self._base)
                    continue
                peer = ctypes.c_void_p()
                rc = lib.awq_b200_peer_region_open(handles[r], ctypes.byref(peer))
                if rc != 0:
                    failure = f"rank {self.rank} could not map the region of rank {r} (code {rc})"
                    break
                self._opened.append(peer.value)
                ptrs.append(peer.value)
            # all ranks leave the constructor the same way
            ok = torch.tensor([0 if failure else 1], device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok[0]) == 0:
                for p in self._opened:
                    lib.awq_b200_peer_region_close(ctypes.c_void_p(p))
                self._opened = []
                dist.barrier(group=group)
                if self._base is not None:
                    lib.awq_b200_peer_region_destroy(ctypes.c_void_p(self._base))
                self._base = None
                raise RuntimeError(failure or "another rank could not map the regions")
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        # this rank's region as a tensor, so that the GEMM can be given a view of it as `out`
        self.region = torch.as_tensor(_DeviceBytes(self._base, size), device=self.device)
        self.state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.calls = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)   # every region is zeroed and mapped before the first call

    def close(self) -> None:
        """Collective: unmaps the peers' regions, then frees this rank's."""
        if self._base is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._opened:
            self._lib.awq_b200_peer_region_close(ctypes.c_void_p(p))
        self._opened = []
        dist.barrier(group=self.group)
        self.region = None
        self._lib.awq_b200_peer_region_destroy(ctypes.c_void_p(self._base))
        self._base = None

    def fits(self, m: int, n: int) -> bool:
        return 0 < m * n * 2 <= self.max_bytes and (m * n * 2) % 16 == 0

    def partial(self, slot: int, m: int, n: int) -> torch.Tensor:
        """This rank's fp16 [m, n] partial inside its region (what the GEMM writes)."""
        off = self.off1 if slot else self.off0
        return self.region[off:off + m * n * 2].view(torch.float16).view(m, n)

    def reduce(self, slot: int, m: int, n: int, out: torch.Tensor | None = None,
               end_barrier: bool = False, dependent_launch: bool = False) -> torch.Tensor:
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
        return self.reduce(slot, m, n)
