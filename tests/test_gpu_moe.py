"""Parity of the router, the token->expert permutation and the fused expert GEMMs with the CPU
oracle."""
import numpy as np
import pytest
import torch

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def A(built_library):
    import awq_b200
    assert torch.cuda.is_available()
    return awq_b200


@pytest.mark.parametrize("t,e,k,renorm,dtype", [
    (1, 128, 8, True, torch.float32), (16, 128, 8, True, torch.float32),
    (333, 128, 8, False, torch.float32), (7, 8, 2, True, torch.float16),
    (5, 1000, 32, True, torch.float32), (4096, 128, 8, True, torch.float32),
])
def test_topk_softmax(A, t, e, k, renorm, dtype):
    g = torch.randn(t, e, generator=torch.Generator().manual_seed(t + e)).to(dtype)
    hs = torch.empty(t, 4, dtype=torch.float16, device="cuda")
    w, ids, tok = A.fused_topk(hs, g.cuda(), k, renorm)
    rw, rids, rtok = O.topk_softmax(g.float().numpy(), k, renorm)
    assert np.array_equal(ids.cpu().numpy(), rids)          # indices bit-exact
    assert np.array_equal(tok.cpu().numpy(), rtok)
    assert np.allclose(w.cpu().numpy(), rw, rtol=2e-5, atol=1e-7)


def test_topk_ties_pick_lower_id(A):
    g = torch.zeros(3, 128)
    g[1, 100] = 1.0
    hs = torch.empty(3, 4, dtype=torch.float16, device="cuda")
    _, ids, _ = A.fused_topk(hs, g.cuda(), 8, True)
    assert ids[0].tolist() == list(range(8))
    assert ids[1].tolist() == [100] + list(range(7))


@pytest.mark.parametrize("t,k,e,blk", [
    (1, 8, 128, 16), (16, 8, 128, 16), (128, 8, 128, 16), (1024, 8, 128, 16), (4096, 8, 128, 16),
    (4, 3, 4, 4), (33, 2, 8, 4), (100, 1, 1000, 8), (64, 8, 128, 64),
])
def test_moe_align_bit_exact(A, t, k, e, blk):
    rng = np.random.default_rng(t * 31 + e)
    ids = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.int32)
    s, eid, post = A.moe_align_block_size(torch.from_numpy(ids).cuda(), blk, e)
    rs, reid, rpost = O.moe_align_block_size(ids, blk, e)
    assert np.array_equal(post.cpu().numpy(), rpost)
    assert np.array_equal(s.cpu().numpy(), rs)
    assert np.array_equal(eid.cpu().numpy(), reid)


def test_moe_align_docstring_example(A, golden):
    ids = torch.from_numpy(golden["align.topk_ids"]).cuda()
    s, eid, post = A.moe_align_block_size(ids, 4, 4)
    assert post.item() == 16
    assert s[:16].cpu().tolist() == golden["align.sorted_ids"].tolist()
    assert eid[:4].cpu().tolist() == [0, 1, 2, 3]


def test_moe_align_expert_map(A):
    rng = np.random.default_rng(9)
    t, k, e, blk = 50, 4, 16, 8
    ids = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.int32)
    emap = np.full(e, -1, dtype=np.int32)
    emap[4:8] = np.arange(4)
    s, eid, post = A.moe_align_block_size(torch.from_numpy(ids).cuda(), blk, e,
                                          torch.from_numpy(emap).cuda(),
                                          ignore_invalid_experts=True)
    rs, reid, rpost = O.moe_align_block_size(ids, blk, e, emap)
    assert np.array_equal(post.cpu().numpy(), rpost)
    assert np.array_equal(s.cpu().numpy(), rs)
    assert np.array_equal(eid.cpu().numpy(), reid)


def test_moe_align_against_installed_vllm(A):
    try:
        from vllm.model_executor.layers.fused_moe.moe_align_block_size import (
            moe_align_block_size as v_align)
        import vllm._moe_C  # noqa: F401
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm compiled ops unavailable: {e}")
    rng = np.random.default_rng(4)
    t, k, e, blk = 200, 8, 128, 16
    ids = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.int32)
    idt = torch.from_numpy(ids).cuda()
    s, eid, post = A.moe_align_block_size(idt, blk, e)
    vs, veid, vpost = v_align(idt, blk, e)
    assert post.item() == vpost.item()
    nb = post.item() // blk
    assert torch.equal(eid[:nb], veid[:nb])
    # same set of pairs per expert; the order inside an expert's run is ours (ascending)
    a = s[:post.item()].cpu().numpy().reshape(nb, blk)
    b = vs[:post.item()].cpu().numpy().reshape(nb, blk)
    ee = eid[:nb].cpu().numpy()
    for x in np.unique(ee):
        assert sorted(a[ee == x].reshape(-1).tolist()) == sorted(b[ee == x].reshape(-1).tolist())


def _moe_case(e, h, i, t, k, seed):
    from awq_b200 import synth
    w1, w2 = synth.moe_layer_tensors(e, h, i, 128, seed=seed)
    x = synth.activations(t, h, seed=seed + 1)
    logits = synth.gating_logits(t, e, seed=seed + 2)
    return w1, w2, x, logits


@pytest.mark.parametrize("e,h,i,t,k", [
    (4, 256, 128, 5, 2), (8, 512, 256, 1, 2), (16, 2048, 768, 16, 8), (128, 2048, 768, 1, 8),
    (128, 2048, 768, 40, 8), (8, 256, 128, 300, 2), (8, 512, 256, 777, 2),
    (128, 2048, 768, 128, 8), (128, 2048, 768, 1024, 8), (128, 2048, 768, 4096, 8),
    # 8-row blocks with experts that need several blocks, and 16-row blocks
    (16, 512, 256, 60, 2), (128, 2048, 768, 200, 8), (8, 256, 128, 50, 2),
])
def test_fused_experts_vs_oracle(A, e, h, i, t, k):
    w1, w2, x, logits = _moe_case(e, h, i, t, k, seed=e + t)
    w, ids, _ = O.topk_softmax(logits.numpy(), k, True)
    ref = O.fused_experts_fp32(x.numpy(), *[a.numpy() for a in w1], *[a.numpy() for a in w2],
                               w, ids)
    w1d = tuple(a.cuda() for a in w1)
    w2d = tuple(a.cuda() for a in w2)
    y = A.fused_experts(x.cuda(), w1d, w2d, torch.from_numpy(w).cuda(),
                        torch.from_numpy(ids).cuda())
    torch.cuda.synchronize()
    y = y.cpu().numpy()
    err = O.rel_err(y, ref)
    assert err < TOL, f"rel err {err}"
    # whole layer through the router as well
    y2 = A.fused_moe(x.cuda(), w1d, w2d, logits.cuda(), k, True).cpu().numpy()
    assert O.rel_err(y2, ref) < TOL


@pytest.mark.parametrize("t,k,e,h,i", [(1, 8, 128, 2048, 768), (2, 8, 128, 2048, 768),
                                       (3, 4, 16, 512, 256), (1, 2, 8, 256, 128),
                                       (4, 8, 128, 2048, 768), (8, 8, 128, 2048, 768),
                                       (5, 8, 16, 8192, 256), (64, 1, 64, 8192, 256),
                                       (64, 1, 16, 512, 256)])
def test_direct_mode_for_a_handful_of_pairs_equals_the_permuted_path(A, t, k, e, h, i, monkeypatch):
    """A handful of (token, slot) pairs skip the permutation kernel (one row block per pair,
    experts read from topk_ids) and the slot sum happens inside the down GEMM (or, when the
    counters do not fit, in the sum kernel).  An identity expert_map forces the permuted path:
    same bits."""
    from awq_b200 import ops
    monkeypatch.setattr(ops, "MOE_DIRECT_MAX_PAIRS", 64)     # the C ABI's limit
    w1, w2, x, logits = _moe_case(e, h, i, t, k, seed=40 + t)
    w1d = tuple(a.cuda() for a in w1)
    w2d = tuple(a.cuda() for a in w2)
    wts, ids, _ = A.fused_topk(x.cuda(), logits.cuda(), k, True)
    direct = A.fused_experts(x.cuda(), w1d, w2d, wts, ids)
    permuted = A.fused_experts(x.cuda(), w1d, w2d, wts, ids, global_num_experts=e,
                               expert_map=torch.arange(e, dtype=torch.int32, device="cuda"))
    assert torch.equal(direct, permuted)
    # two slots of one token on the same expert: the pair blocks stay independent
    if k == 1:
        return
    ids2 = ids.clone()
    ids2[:, 1] = ids2[:, 0]
    direct2 = A.fused_experts(x.cuda(), w1d, w2d, wts, ids2)
    permuted2 = A.fused_experts(x.cuda(), w1d, w2d, wts, ids2, global_num_experts=e,
                                expert_map=torch.arange(e, dtype=torch.int32, device="cuda"))
    assert torch.equal(direct2, permuted2)
    ref = O.fused_experts_fp32(x.numpy(), *[a.numpy() for a in w1], *[a.numpy() for a in w2],
                               wts.cpu().numpy(), ids2.cpu().numpy())
    assert O.rel_err(direct2.float().cpu().numpy(), ref) < TOL


def test_wna16_layout_converts_back_bit_exact(A, golden):
    """uint8 [E, N, K/2] (vLLM's MoE WNA16 layout) -> AWQ layout on the device: vLLM's own
    converted tensors give back the AWQ tensors they were made from, and stacked random experts
    agree with the oracle's conversion."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                             "wna16_golden.npz"))
    for name in ("small", "wide", "g64"):
        grp = int(g[f"{name}.group"][0])
        q, s, z = A.wna16_to_awq(torch.from_numpy(g[f"{name}.wna16_qweight"])[None].cuda(),
                                 torch.from_numpy(g[f"{name}.wna16_scales"])[None].cuda(),
                                 torch.from_numpy(g[f"{name}.wna16_qzeros"])[None].cuda(), grp)
        assert np.array_equal(q[0].cpu().numpy(), g[f"{name}.qweight"])
        assert np.array_equal(z[0].cpu().numpy(), g[f"{name}.qzeros"])
        assert np.array_equal(s[0].cpu().numpy(), g[f"{name}.scales"])
    w1, w2, _, _ = _moe_case(6, 384, 160, 1, 2, seed=3)     # ragged tiles: N = 320 / 384, K = 384 / 160
    for qw, sc, qz in (w1, w2):
        wu = np.stack([O.awq_to_wna16_qweight(a) for a in qw.numpy()])
        zu = np.stack([O.awq_to_wna16_qzeros(a) for a in qz.numpy()])
        su = np.ascontiguousarray(sc.numpy().transpose(0, 2, 1))
        grp = qw.shape[1] // sc.shape[1]
        q, s, z = A.wna16_to_awq(torch.from_numpy(wu).cuda(), torch.from_numpy(su).cuda(),
                                 torch.from_numpy(zu).cuda(), grp)
        assert torch.equal(q.cpu(), qw) and torch.equal(z.cpu(), qz) and torch.equal(s.cpu(), sc)


def test_fused_experts_accepts_the_reference_call_form(A):
    """w1 / w2 as the stacked qweight tensors plus a quant_config object carrying scales and zero
    points (vLLM fused_moe.py:1587-1599) gives the same bits as the triple form."""
    from types import SimpleNamespace
    e, h, i, t, k = 16, 512, 256, 33, 4
    w1, w2, x, logits = _moe_case(e, h, i, t, k, seed=5)
    w1d = tuple(a.cuda() for a in w1)
    w2d = tuple(a.cuda() for a in w2)
    wts, ids, _ = A.fused_topk(x.cuda(), logits.cuda(), k, True)
    y = A.fused_experts(x.cuda(), w1d, w2d, wts, ids)
    qc = SimpleNamespace(w1_scale=w1d[1], w2_scale=w2d[1], w1_zp=w1d[2], w2_zp=w2d[2],
                         block_shape=[0, 128])
    y2 = A.fused_experts(x.cuda(), w1d[0], w2d[0], wts, ids, quant_config=qc)
    assert torch.equal(y, y2)
    with pytest.raises(ValueError):
        A.fused_experts(x.cuda(), w1d[0], w2d[0], wts, ids)
    with pytest.raises(ValueError):
        A.fused_experts(x.cuda(), w1d[0], w2d[0], wts, ids,
                        quant_config=SimpleNamespace(w1_scale=w1d[1], w2_scale=w2d[1],
                                                     w1_zp=None, w2_zp=None))


@pytest.mark.parametrize("t", [20, 400])
def test_fused_experts_expert_parallel_shards_sum(A, t):
    """Two expert-parallel shards (expert_map) add up to the unsharded layer (T = 20: streaming
    kernels, T = 400: grouped tcgen05 GEMMs with blocks of experts that live on another rank)."""
    e, h, i, k = 8, 256, 128, 2
    w1, w2, x, logits = _moe_case(e, h, i, t, k, seed=77)
    w, ids, _ = O.topk_softmax(logits.numpy(), k, True)
    wt, idt = torch.from_numpy(w).cuda(), torch.from_numpy(ids).cuda()
    full = A.fused_experts(x.cuda(), tuple(a.cuda() for a in w1), tuple(a.cuda() for a in w2),
                           wt, idt).float()
    acc = torch.zeros_like(full)
    for lo in (0, 4):
        emap = torch.full((e,), -1, dtype=torch.int32)
        emap[lo:lo + 4] = torch.arange(4, dtype=torch.int32)
        w1s = tuple(a[lo:lo + 4].contiguous().cuda() for a in w1)
        w2s = tuple(a[lo:lo + 4].contiguous().cuda() for a in w2)
        acc += A.fused_experts(x.cuda(), w1s, w2s, wt, idt, global_num_experts=e,
                               expert_map=emap.cuda()).float()
    assert O.rel_err(acc.cpu().numpy(), full.cpu().numpy()) < 5e-3


def test_fused_moe_full_size_rows_are_independent(A):
    """Benchmark-size check without the oracle: a token's output does not depend on which other
    tokens share the batch, so the first rows of the T = 4096 layer (tcgen05 grouped GEMMs)
    must match the same tokens run as a T = 48 batch (weight-streaming kernels)."""
    e, h, i, k = 128, 2048, 768, 8
    w1, w2, x, logits = _moe_case(e, h, i, 4096, k, seed=123)
    w1d = tuple(a.cuda() for a in w1)
    w2d = tuple(a.cuda() for a in w2)
    big = A.fused_moe(x.cuda(), w1d, w2d, logits.cuda(), k, True)
    small = A.fused_moe(x[:48].cuda().contiguous(), w1d, w2d, logits[:48].cuda().contiguous(), k, True)
    torch.cuda.synchronize()
    assert torch.isfinite(big.float()).all()
    assert O.rel_err(big[:48].cpu().numpy(), small.float().cpu().numpy()) < 5e-3


@pytest.mark.parametrize("t,h,i,e,k", [(1, 2048, 768, 128, 8), (16, 2048, 768, 128, 8),
                                       (8, 256, 128, 50, 2), (40, 512, 256, 12, 2),
                                       (256, 2048, 768, 128, 8), (300, 512, 256, 4, 2)])
def test_experts_on_decode_layout_copies_equal_checkpoint_layout(A, t, h, i, e, k):
    """fused_experts with the decode-layout copies of the expert weights: bit-identical to the
    checkpoint layout where the streaming kernels run (blocks of 8 / 16 rows), and the copies
    are simply not used where the grouped tcgen05 GEMMs run (last case)."""
    from awq_b200 import synth
    w1, w2 = synth.moe_layer_tensors(e, h, i, 128, seed=t + e)
    w1 = tuple(a.cuda() for a in w1)
    w2 = tuple(a.cuda() for a in w2)
    x = synth.activations(t, h, seed=t).cuda()
    logits = synth.gating_logits(t, e, seed=e).cuda()
    w, ids, _ = A.fused_topk(x, logits, k, True)
    d1, d2 = A.awq_repack(w1[0]), A.awq_repack(w2[0])
    assert d1.shape == w1[0].shape and d2.shape == w2[0].shape
    y0 = A.fused_experts(x, w1, w2, w, ids)
    y1 = A.fused_experts(x, w1, w2, w, ids, w1_decode=d1, w2_decode=d2)
    torch.cuda.synchronize()
    assert torch.equal(y0, y1)
    ref = O.fused_experts_fp32(x.cpu().numpy(), *[a.cpu().numpy() for a in w1],
                          *[a.cpu().numpy() for a in w2], w.cpu().numpy(), ids.cpu().numpy(), 128)
    assert O.rel_err(y1.cpu().numpy(), ref) < TOL
    with pytest.raises(ValueError):
        A.fused_experts(x, w1, w2, w, ids, w1_decode=d1)
