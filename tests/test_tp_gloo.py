"""Tensor-parallel sharding and the row-parallel exchange step on CPU: two gloo ranks.  The
per-rank products are computed by the oracle (the checker); the code under test is the
sharding, padding and all-reduce logic of awq_b200.tp."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, k, n, results):
    for p in (ROOT, os.path.join(ROOT, "server-benchmark_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from awq_b200 import synth, tp
    from oracle import awq_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=5)
        x = synth.activations(4, k, seed=6)
        full = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy())
        # row-parallel: pad K to a multiple of world groups, shard, partial product, all-reduce
        pqw, ps, pqz = tp.pad_k_for_tp(qw, s, qz, world)
        assert ps.shape[0] % world == 0
        sh = tp.shard_rows(pqw, ps, pqz, rank, world)
        xs = tp.shard_input(tp.pad_x_for_tp(x, pqw.shape[0]), rank, world)
        assert sh[0].shape[0] == xs.shape[1] and sh[0].shape[0] % 128 == 0
        part = torch.from_numpy(O.awq_gemm_fp32(xs.numpy(), *[a.numpy() for a in sh]))
        y = tp.all_reduce_output(part)
        ok_row = np.allclose(y.numpy(), full, rtol=1e-4, atol=1e-3)
        # column-parallel: shards concatenate to the full output
        shc = tp.shard_columns(qw, s, qz, rank, world)
        yc = torch.from_numpy(O.awq_gemm_fp32(x.numpy(), *[a.numpy() for a in shc]))
        gathered = [torch.empty_like(yc) for _ in range(world)]
        dist.all_gather(gathered, yc)
        ok_col = np.allclose(torch.cat(gathered, dim=1).numpy(), full, rtol=1e-4, atol=1e-3)
        results[rank] = (ok_row, ok_col)
    finally:
        dist.destroy_process_group()


def test_tp_shards_two_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    # K = 3 groups: not divisible by 2 -> exercises the zero-group padding
    mp.spawn(_worker, args=(world, port, 384, 64, results), nprocs=world, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}


def test_shard_validation():
    sys.path.insert(0, os.path.join(ROOT, "server-benchmark_b200"))
    from awq_b200 import synth, tp
    qw, s, qz = synth.awq_linear_tensors(384, 64, 128, seed=1)
    with pytest.raises(ValueError, match="input size is not aligned"):
        tp.shard_rows(qw, s, qz, 0, 2)
    with pytest.raises(ValueError, match="output size is not aligned"):
        tp.shard_columns(qw, s, qz, 0, 3)
    a = tp.shard_columns(qw, s, qz, 1, 2)
    assert a[0].shape == (384, 4) and a[1].shape == (3, 32) and a[2].shape == (3, 4)
    assert torch.equal(a[1], s[:, 32:])
