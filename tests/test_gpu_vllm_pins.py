"""Second pin of the MoE half of the oracle, and of the dense path, against the installed vLLM's
own compiled kernels on the same GPU (awq_b200/vllm_ref.py): the router kernel
(torch.ops._moe_C.topk_softmax), the default AWQ expert path (fused_marlin_moe after vLLM's own
AWQ -> Marlin conversion) and the default dense route (awq_marlin_repack + marlin_gemm).
Skipped only when vLLM's compiled ops do not load."""
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


@pytest.fixture(scope="module")
def V():
    from awq_b200 import vllm_ref
    if not vllm_ref.available():
        pytest.skip(f"vllm compiled ops unavailable: {vllm_ref.why_unavailable()}")
    return vllm_ref


@pytest.mark.parametrize("t,e,k,renorm", [(1, 128, 8, True), (16, 128, 8, True),
                                          (333, 128, 8, False), (4096, 128, 8, True),
                                          (7, 64, 4, True)])
def test_router_against_vllm_kernel(A, V, t, e, k, renorm):
    g = torch.randn(t, e, generator=torch.Generator().manual_seed(t * 7 + e)).cuda()
    hs = torch.empty(t, 4, dtype=torch.float16, device="cuda")
    w, ids, _ = A.fused_topk(hs, g, k, renorm)
    vw, vids = V.topk_softmax(g, k, renorm)
    assert torch.equal(ids, vids)                                   # expert ids exact
    assert torch.allclose(w, vw, rtol=2e-5, atol=1e-7)
    # and the oracle agrees with both
    rw, rids, _ = O.topk_softmax(g.cpu().numpy(), k, renorm)
    assert np.array_equal(rids, vids.cpu().numpy())
    assert np.allclose(rw, vw.cpu().numpy(), rtol=2e-5, atol=1e-7)


def test_router_tie_rule_matches_vllm(A, V):
    """Equal logits: the oracle and this package take the lower expert id first; vLLM's kernel
    must do the same for the pin to hold on ties."""
    g = torch.zeros(4, 128)
    g[1, 100] = 1.0
    g[2, 5:9] = 2.0
    g[3, ::2] = -1.0
    g = g.cuda()
    hs = torch.empty(4, 4, dtype=torch.float16, device="cuda")
    _, ids, _ = A.fused_topk(hs, g, 8, True)
    _, vids = V.topk_softmax(g, 8, True)
    assert torch.equal(ids, vids)


@pytest.mark.parametrize("t", [1, 16, 128, 1024])
def test_experts_against_vllm_marlin_moe(A, V, t):
    """Qwen3-30B-A3B expert shapes, identical AWQ tensors: this package's fused experts, vLLM's
    fused_marlin_moe on its own repack of them, and the fp32 oracle agree within tolerance."""
    from awq_b200 import synth
    e, h, i, k = 128, 2048, 768, 8
    w1, w2 = synth.moe_layer_tensors(e, h, i, 128, seed=3)
    x = synth.activations(t, h, seed=4)
    logits = synth.gating_logits(t, e, seed=5)
    w, ids, _ = O.topk_softmax(logits.numpy(), k, True)
    wt, idt = torch.from_numpy(w).cuda(), torch.from_numpy(ids).cuda()
    w1d, w2d = tuple(a.cuda() for a in w1), tuple(a.cuda() for a in w2)
    ours = A.fused_experts(x.cuda(), w1d, w2d, wt, idt).float().cpu().numpy()
    prepared = V.marlin_moe_prepare(w1d, w2d)
    theirs = V.marlin_moe(x.cuda(), prepared, wt, idt).float().cpu().numpy()
    assert O.rel_err(ours, theirs) < TOL
    if t <= 128:
        ref = O.fused_experts_fp32(x.numpy(), *[a.numpy() for a in w1], *[a.numpy() for a in w2],
                                   w, ids)
        assert O.rel_err(ours, ref) < TOL
        assert O.rel_err(theirs, ref) < TOL   # vLLM's own path is inside the oracle's tolerance


@pytest.mark.parametrize("m,k,n", [(1, 8192, 8192), (16, 8192, 8192), (64, 8192, 10240),
                                   (256, 4096, 2048)])
def test_dense_against_vllm_marlin_and_awq_gemm(A, V, m, k, n):
    from awq_b200 import synth
    qw, s, qz = [t.cuda() for t in synth.awq_linear_tensors(k, n, 128, seed=m)]
    x = synth.activations(m, k, seed=m + 1).cuda()
    ours = A.awq_gemm(x, qw, s, qz, 8).float().cpu().numpy()
    marlin = V.marlin_gemm(x, V.marlin_prepare(qw, s, qz)).float().cpu().numpy()
    assert O.rel_err(ours, marlin) < TOL
    if m < 256:
        # vLLM's own kernel only while the plug-in has not re-implemented the op in this process
        # (test files that register it are named to run after this one)
        from awq_b200 import vllm_plugin
        assert not vllm_plugin._registered, "plug-in registered before the pins ran"
        theirs = V.awq_gemm(x, qw, s, qz).float().cpu().numpy()
        assert O.rel_err(ours, theirs) < TOL
