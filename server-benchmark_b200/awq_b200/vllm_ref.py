"""The installed vLLM's own kernels for the same work, on the same GPU: the bars the kernels of
this package are measured against and a second pin for the CPU oracle.

Nothing here is on the product path: ``bench.py`` times these calls next to ours and the GPU
tests compare results.  Everything is called through vLLM's public Python wrappers (paths
inside the ``vllm`` package):

  awq_gemm / awq_dequantize          _custom_ops.py:542-605 (what AWQLinearMethod.apply calls)
  awq_marlin_repack + marlin_gemm    quantization/utils/marlin_utils.py:577-640,
                                     quantization/awq_marlin.py:379-507 (the default dense route)
  fused_marlin_moe                   fused_moe/experts/marlin_moe.py:225-262 with the weight
                                     conversion of fused_moe/oracle/int_wna16.py:385-527 (the
                                     default AWQ MoE route)
  topk_softmax                       _custom_ops.py:2370-2385

``available()`` says whether the compiled ops load (they need a CUDA driver).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

_state: dict = {}


def available() -> bool:
    if "ok" not in _state:
        try:
            import vllm._C  # noqa: F401
            import vllm._moe_C  # noqa: F401
            _state["ok"] = True
        except Exception as e:  # pragma: no cover - depends on the box
            _state["ok"] = False
            _state["why"] = f"{type(e).__name__}: {e}"
    return _state["ok"]


def why_unavailable() -> str:
    available()
    return _state.get("why", "")


# ------------------------------------------------------------------ dense


def awq_gemm(x, qweight, scales, qzeros, split_k_iters: int = 8):
    """torch.ops._C.awq_gemm as vLLM registers it (must be called before the plug-in overrides
    it, or with the plug-in not registered)."""
    return torch.ops._C.awq_gemm(x, qweight, scales, qzeros, split_k_iters)


def awq_dequant_matmul(x, qweight, scales, qzeros):
    """The >= 256-token route of AWQLinearMethod.apply (awq.py:276-281)."""
    w = torch.ops._C.awq_dequantize(qweight, scales, qzeros, 0, 0, 0)
    return torch.matmul(x, w)


@dataclass
class MarlinLinear:
    qweight: torch.Tensor
    scales: torch.Tensor
    zeros: torch.Tensor
    g_idx: torch.Tensor
    workspace: torch.Tensor
    n: int
    k: int


def marlin_prepare(qweight, scales, qzeros, group: int = 128) -> MarlinLinear:
    """AWQ checkpoint tensors -> Marlin layout, the way AWQMarlinLinearMethod does at load time
    (awq_marlin.py:456-499)."""
    from vllm import _custom_ops as vops
    from vllm.model_executor.layers.quantization.utils import marlin_utils as mu

    k, n = qweight.shape[0], qweight.shape[1] * 8
    dev = qweight.device
    mq = vops.awq_marlin_repack(qweight, size_k=k, size_n=n, num_bits=4)
    ms = mu.marlin_permute_scales(scales, size_k=k, size_n=n, group_size=group)
    mz = mu.awq_to_marlin_zero_points(qzeros, size_k=k // group, size_n=n, num_bits=4)
    return MarlinLinear(mq, ms, mz, mu.marlin_make_empty_g_idx(dev),
                        mu.marlin_make_workspace_new(dev), n, k)


def marlin_gemm(x, m: MarlinLinear):
    from vllm.model_executor.layers.quantization.utils import marlin_utils as mu
    from vllm.scalar_type import scalar_types

    return mu.apply_awq_marlin_linear(x, m.qweight, m.scales, m.zeros, m.g_idx, m.g_idx,
                                      m.workspace, scalar_types.uint4, m.n, m.k)


# ------------------------------------------------------------------ MoE


def topk_softmax(gating: torch.Tensor, topk: int, renormalize: bool):
    """vLLM's router kernel on fp32 logits: (weights f32 [T,k], ids i32 [T,k])."""
    from vllm import _custom_ops as vops

    t = gating.shape[0]
    w = torch.empty(t, topk, dtype=torch.float32, device=gating.device)
    ids = torch.empty(t, topk, dtype=torch.int32, device=gating.device)
    tok = torch.empty(t, topk, dtype=torch.int32, device=gating.device)
    try:
        vops.topk_softmax(w, ids, tok, gating.float().contiguous(), renormalize)
    except TypeError:
        vops.topk_softmax(w, ids, tok, gating.float().contiguous())
        if renormalize:
            w = w / w.sum(dim=-1, keepdim=True)
    return w, ids


@dataclass
class MarlinMoE:
    w13: torch.Tensor
    w2: torch.Tensor
    s13: torch.Tensor
    s2: torch.Tensor
    z13: torch.Tensor
    z2: torch.Tensor
    sort13: torch.Tensor
    sort2: torch.Tensor
    workspace: torch.Tensor


def marlin_moe_prepare(w1, w2, group: int = 128) -> MarlinMoE:
    """Stacked AWQ expert tensors -> Marlin MoE layout, following
    fused_moe/oracle/int_wna16.py:385-527 step by step."""
    from vllm import _custom_ops as vops
    from vllm.model_executor.layers.quantization.utils import marlin_utils as mu

    (w13_q, w13_s, w13_z), (w2_q, w2_s, w2_z) = w1, w2
    e = w13_q.shape[0]
    dev = w13_q.device
    inter = w2_q.shape[1]
    sort13 = torch.empty((e, 0), dtype=torch.int32, device=dev)
    sort2 = torch.empty((e, 0), dtype=torch.int32, device=dev)
    m13 = vops.awq_marlin_moe_repack(w13_q, sort13, size_k=w13_q.shape[1],
                                     size_n=w13_q.shape[2] * 8, num_bits=4)
    m2 = vops.awq_marlin_moe_repack(w2_q, sort2, size_k=w2_q.shape[1],
                                    size_n=w2_q.shape[2] * 8, num_bits=4)
    s13 = mu.marlin_moe_permute_scales(s=w13_s, size_k=inter, size_n=w13_s.shape[2],
                                       group_size=group)
    s2 = mu.marlin_moe_permute_scales(s=w2_s, size_k=inter, size_n=w2_s.shape[2],
                                      group_size=group)
    z13 = mu.moe_awq_to_marlin_zero_points(w13_z, size_k=w13_z.shape[1],
                                           size_n=w13_z.shape[2] * 8, num_bits=4)
    z2 = mu.moe_awq_to_marlin_zero_points(w2_z, size_k=w2_z.shape[1],
                                          size_n=w2_z.shape[2] * 8, num_bits=4)
    return MarlinMoE(m13, m2, s13, s2, z13, z2, sort13, sort2,
                     mu.marlin_make_workspace_new(dev, 4))


def marlin_moe(x, m: MarlinMoE, topk_weights, topk_ids):
    from vllm.model_executor.layers.fused_moe.experts.marlin_moe import fused_marlin_moe
    from vllm.scalar_type import scalar_types

    return fused_marlin_moe(x, m.w13, m.w2, None, None, m.s13, m.s2, topk_weights, topk_ids,
                            quant_type_id=scalar_types.uint4.id,
                            global_num_experts=m.w13.shape[0],
                            sort_indices1=m.sort13, sort_indices2=m.sort2,
                            w1_zeros=m.z13, w2_zeros=m.z2, workspace=m.workspace,
                            is_k_full=True)
