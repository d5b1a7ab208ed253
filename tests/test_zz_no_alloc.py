"""awq_b200_moe_experts_static: the fused-MoE expert GEMMs for hosts that cannot get device
memory at call time (an engine whose KV-cache pool already owns all free HBM, a C / FFI host
without a device allocator).  The scratch the expert kernels need sits in a 16 MiB array inside
the library instead of a caller buffer.

The test drives the entry point through the C ABI and compares it with awq_b200_moe_experts (which
takes the scratch from the caller) on the same inputs, twice in a row with different inputs, so
that stale contents of the shared array would show.  It also checks the size limit.
This file is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(lib, e, h, i, t, k, seed):
    from awq_b200 import synth
    import awq_b200
    w1, w2 = synth.moe_layer_tensors(e, h, i, 128, seed=seed)
    w1 = tuple(a.cuda() for a in w1)
    w2 = tuple(a.cuda() for a in w2)
    x = synth.activations(t, h, seed=seed + 1).cuda()
    logits = synth.gating_logits(t, e, seed=seed + 2).cuda()
    wts, ids, _ = awq_b200.fused_topk(x, logits, k, True)
    block = lib.awq_b200_moe_block_size(t, k, e, h, i, 128)
    sorted_ids, expert_ids, num_post = awq_b200.moe_align_block_size(ids, block, e)
    return dict(x=x, w1=w1, w2=w2, wts=wts, sorted_ids=sorted_ids, expert_ids=expert_ids,
                num_post=num_post, block=block, dims=(t, k, e, h, i))


def _common_args(p, out):
    t, k, e, h, i = p["dims"]
    ptrs = [p["x"], *p["w1"], *p["w2"], p["wts"], p["sorted_ids"], p["expert_ids"],
            p["num_post"], out]
    return [a.data_ptr() for a in ptrs] + [t, k, e, h, i, 128, p["block"], 0,
                                           p["sorted_ids"].numel()]


def _run_both(lib, p):
    t, k, e, h, i = p["dims"]
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.awq_b200_moe_workspace_bytes(t, k, e, h, i)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    out_ref = torch.full((t, h), float("nan"), dtype=torch.float16, device="cuda")
    out_new = torch.full((t, h), float("nan"), dtype=torch.float16, device="cuda")
    rc = lib.awq_b200_moe_experts(*_common_args(p, out_ref), ws.data_ptr(), need, stream)
    assert rc == 0
    rc = lib.awq_b200_moe_experts_static(*_common_args(p, out_new), stream)
    assert rc == 0
    torch.cuda.synchronize()
    return out_ref, out_new


def test_static_scratch_entry_point_matches_caller_scratch_twice(built_library):
    from awq_b200 import _lib
    lib = _lib.load()
    assert lib.awq_b200_moe_static_scratch_bytes() == 16 << 20
    # two different problems back to back: the second call starts from the first one's leftovers
    for seed, (e, h, i, t, k) in [(3, (16, 512, 256, 24, 4)), (9, (8, 256, 128, 7, 2))]:
        p = _problem(lib, e, h, i, t, k, seed)
        out_ref, out_new = _run_both(lib, p)
        assert torch.isfinite(out_new.float()).all()
        # same kernels, same launch geometry, scratch in a different place: identical bits
        assert torch.equal(out_ref, out_new)
        # and the same tolerance against the oracle as the other MoE tests
        from awq_b200 import synth
        from oracle import awq_oracle as O
        logits = synth.gating_logits(t, e, seed=seed + 2)
        w, ids, _ = O.topk_softmax(logits.numpy(), k, True)
        w1, w2 = synth.moe_layer_tensors(e, h, i, 128, seed=seed)
        xr = synth.activations(t, h, seed=seed + 1)
        ref = O.fused_experts_fp32(xr.numpy(), *[a.numpy() for a in w1],
                                   *[a.numpy() for a in w2], w, ids)
        assert O.rel_err(out_new.cpu().numpy(), ref) < 1e-2


def test_static_scratch_entry_point_refuses_oversized_problems(built_library):
    from awq_b200 import _lib
    lib = _lib.load()
    t, k, e, h, i = 4096, 8, 128, 2048, 768
    assert lib.awq_b200_moe_workspace_bytes(t, k, e, h, i) > lib.awq_b200_moe_static_scratch_bytes()
    buf = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    cap = lib.awq_b200_moe_sorted_capacity(t * k, e, 16)
    rc = lib.awq_b200_moe_experts_static(p, p, p, p, p, p, p, p, p, p, p, p, t, k, e, h, i, 128, 16,
                                         0, cap, None)
    assert rc == -9
    assert "capacity" in _lib.strerror(rc)
