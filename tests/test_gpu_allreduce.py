"""awq_b200_allreduce through the C ABI: the one-rank case, the give-up path of its bounded
waits (a peer flag that nobody sets; the kernel returns, the status word says which wait), and,
where two GPUs are visible, two ranks as child processes against NCCL's all-reduce, eager and
replayed from a CUDA graph."""
import ctypes
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _status(lib) -> int:
    v = ctypes.c_int(-1)
    assert lib.awq_b200_device_status_clear(ctypes.byref(v)) == 0
    return v.value


def test_single_rank_is_a_copy(built_library):
    from awq_b200 import _lib, tp
    lib = _lib.load()
    m, n = 16, 8192
    off0, _, size = tp.region_layout(m * n * 2)
    region = torch.zeros(size, dtype=torch.uint8, device="cuda")
    x = torch.randn(m, n, device="cuda").half()
    region[off0:off0 + m * n * 2].view(torch.float16).view(m, n).copy_(x)
    out = torch.empty_like(x)
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 1)(region.data_ptr())
    for call in range(3):
        rc = lib.awq_b200_allreduce(ptrs, 0, 1, off0, out.data_ptr(), m * n * 2,
                                    state.data_ptr(), call & 1, None)
        assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(out, x)
    assert state.tolist() == [3, 0]          # three calls numbered on the device
    assert _status(lib) == 0
    # argument checks happen before any launch
    assert lib.awq_b200_allreduce(ptrs, 0, 9, off0, out.data_ptr(), 32, state.data_ptr(), 0,
                                  None) < 0   # more ranks than the kernel takes
    assert lib.awq_b200_allreduce(ptrs, 0, 1, 16, out.data_ptr(), 32, state.data_ptr(), 0,
                                  None) < 0   # data inside the flag area


def test_wait_for_a_silent_peer_runs_out(built_library):
    """World of two whose second region is plain local memory that nobody else touches: the
    start barrier never completes, the wait gives up after the (tiny) limit, the kernel returns
    and the context stays usable."""
    from awq_b200 import _lib, tp
    lib = _lib.load()
    m, n = 4, 1024
    off0, _, size = tp.region_layout(m * n * 2)
    mine = torch.zeros(size, dtype=torch.uint8, device="cuda")
    silent = torch.zeros(size, dtype=torch.uint8, device="cuda")
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), silent.data_ptr())
    lib.awq_b200_set_wait_limit(2000)
    try:
        assert lib.awq_b200_allreduce(ptrs, 0, 2, off0, out.data_ptr(), m * n * 2,
                                      state.data_ptr(), 0, None) == 0
        torch.cuda.synchronize()
        assert _status(lib) == 71                # start barrier, peer 1
        # this rank did publish its own flag into the peer's region before it gave up
        flags = silent[:tp.FLAG_BYTES].view(torch.int32)
        assert int(flags[0]) == 1
    finally:
        lib.awq_b200_set_wait_limit(0)
    # the context still works
    assert torch.equal(out, torch.zeros_like(out))
    assert _status(lib) == 0


TWO_RANKS = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, os.path.join(ROOT, "server-benchmark_b200"))
    import torch, torch.distributed as dist
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from awq_b200 import tp
    comm = tp.PeerAllReduce(256 * 8192 * 2)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    worst = 0.0
    for i, (m, n) in enumerate([(1, 8192), (16, 8192), (7, 1024), (256, 8192), (16, 8192)] * 3):
        x = torch.randn(m, n, device="cuda", generator=gen).half()
        ref = x.clone(); dist.all_reduce(ref)
        got = comm.all_reduce(x)
        torch.cuda.synchronize()
        worst = max(worst, float((got.float() - ref.float()).abs().max()))
    # graph replay: two calls per replay, alternating slots
    xs = [torch.randn(16, 8192, device="cuda", generator=gen).half() for _ in range(2)]
    refs = []
    for x in xs:
        r = x.clone(); dist.all_reduce(r); refs.append(r)
    def step():
        outs = []
        for j, x in enumerate(xs):
            comm.partial(j, 16, 8192).copy_(x)
            outs.append(comm.reduce(j, 16, 8192, dependent_launch=False))
        return outs
    step(); torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        outs = step()
    for _ in range(20):
        g.replay()
    torch.cuda.synchronize()
    for o, r in zip(outs, refs):
        worst = max(worst, float((o.float() - r.float()).abs().max()))
    import ctypes
    from awq_b200 import _lib
    v = ctypes.c_int(-1); _lib.load().awq_b200_device_status_clear(ctypes.byref(v))
    t = torch.tensor([worst, float(v.value)], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print("RESULT", float(t[0]), int(t[1]))
    del g
    comm.close()
    dist.barrier(); dist.destroy_process_group()
""")


def test_two_ranks_against_nccl(built_library, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "two_ranks.py"
    script.write_text(f"ROOT = {ROOT!r}\n" + TWO_RANKS)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                          "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29631", str(script)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, (res.stdout + res.stderr)[-3000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("RESULT")][-1].split()
    # fp16 rounding of a two-term sum: NCCL and the kernel both add in fp32 and round once
    assert float(line[1]) <= 2e-2 and int(line[2]) == 0
