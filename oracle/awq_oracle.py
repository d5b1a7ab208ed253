"""CPU restatement of the AWQ W4A16 linear / fused-MoE arithmetic.

THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are compared with;
it is never imported by the product package.  Only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may use it.

The reference harness (cloudrift-ai/server-benchmark) contains no arithmetic of its own: it
starts the floating docker tag ``vllm/vllm-openai:latest`` (run_remote_benchmark.py:344,
utils/generate_compose.py:67) and measures it over HTTP (benchmarks/3_vllm_benchmark.sh:151-162).
The arithmetic therefore lives in the third-party dependency vLLM.  The copy restated here is
vLLM 0.22.0; every function cites the vLLM file (path inside the ``vllm`` package) it follows.

Pinning: ``tests/golden/make_golden.py`` runs vLLM's own pure-Python packer
(``quant_utils.awq_pack``) and vLLM's own Triton AWQ kernels under the Triton CPU
interpreter and stores inputs and outputs; ``tests/test_oracle.py`` checks this file
against those vectors, against the known word 0x75316420, and against the worked example in
the ``moe_align_block_size`` docstring.

Integer work is numpy; floating point work is numpy/torch fp32.
"""
from __future__ import annotations

import numpy as np

# Nibble p (counted from the least significant nibble) of a packed word holds column
# AWQ_ORDER[p] of the 8 columns the word covers.
# vLLM: model_executor/layers/quantization/utils/quant_utils.py:794-813 (awq_pack interleave
# [0,2,4,6,1,3,5,7]); model_executor/layers/quantization/awq_triton.py:54-67 (inverse,
# shifts 4*[0,4,1,5,2,6,3,7]).
AWQ_ORDER = np.array([0, 2, 4, 6, 1, 3, 5, 7], dtype=np.int64)
# Column j of the 8 lives in nibble AWQ_REVERSE[j].
AWQ_REVERSE = np.array([0, 4, 1, 5, 2, 6, 3, 7], dtype=np.int64)
PACK = 8


def pack_awq(q: np.ndarray) -> np.ndarray:
    """[R, C] integers in 0..15  ->  int32 [R, C/8] in AWQ nibble order.

    vLLM: quant_utils.py:794-813 (awq_pack) followed by :728-751 (pack_cols).
    """
    q = np.asarray(q)
    assert q.ndim == 2 and q.shape[1] % PACK == 0
    assert q.min(initial=0) >= 0 and q.max(initial=0) <= 15
    r, c = q.shape
    g = q.reshape(r, c // PACK, PACK).astype(np.uint32)
    word = np.zeros((r, c // PACK), dtype=np.uint32)
    for p in range(PACK):
        word |= g[:, :, AWQ_ORDER[p]] << np.uint32(4 * p)
    return word.view(np.int32)


def unpack_awq(packed: np.ndarray) -> np.ndarray:
    """int32 [R, C/8]  ->  uint8 [R, C]; q[r, 8c+j] = (word[r,c] >> 4*AWQ_REVERSE[j]) & 0xF.

    vLLM: awq_triton.py:54-67 and :144-153 (shift table and mask).
    """
    w = np.ascontiguousarray(packed).view(np.uint32)
    r, c = w.shape
    out = np.empty((r, c, PACK), dtype=np.uint8)
    for j in range(PACK):
        out[:, :, j] = (w >> np.uint32(4 * AWQ_REVERSE[j])) & np.uint32(0xF)
    return out.reshape(r, c * PACK)


def dequantize_fp32(qweight, scales, qzeros, group: int = 128) -> np.ndarray:
    """W[k, n] = (q[k, n] - z[k // group, n]) * s[k // group, n], evaluated in fp32.

    vLLM: awq_triton.py:70-101 (zero/scale row = k // group, (q - z) * s).
    """
    q = unpack_awq(qweight).astype(np.float32)
    z = unpack_awq(qzeros).astype(np.float32)
    s = np.asarray(scales).astype(np.float32)
    k = q.shape[0]
    assert k % group == 0 and z.shape[0] == k // group and s.shape == z.shape
    return (q - np.repeat(z, group, axis=0)) * np.repeat(s, group, axis=0)


def dequantize_fp16(qweight, scales, qzeros, group: int = 128) -> np.ndarray:
    """The fp16 result ``awq_dequantize`` returns: (q - z) is exact in fp16 and the product
    with the fp16 scale is rounded once (round-to-nearest-even).

    vLLM: awq_triton.py:101 (the expression is evaluated in the scale dtype).
    fp32 holds the exact product of an integer in [-15, 15] and an 11-bit significand, so
    rounding the fp32 product to fp16 is the single rounding the fp16 multiply performs.
    """
    return dequantize_fp32(qweight, scales, qzeros, group).astype(np.float16)


def awq_gemm_fp32(x, qweight, scales, qzeros, group: int = 128) -> np.ndarray:
    """y = x.float() @ dequantize_fp32(...), fp32 result (the caller rounds to fp16).

    This is the "PyTorch fp32 dequantise-then-matmul" definition of the layer.
    vLLM call site: model_executor/layers/quantization/awq.py:276-283.
    """
    import torch

    w = torch.from_numpy(dequantize_fp32(qweight, scales, qzeros, group))
    xt = torch.from_numpy(np.asarray(x).astype(np.float32))
    return (xt @ w).numpy()


def awq_gemm_fp32_torch(x, qweight, scales, qzeros, group: int = 128):
    """The same dequantise-then-matmul written with torch tensor ops only (torch CPU tensors in,
    fp32 torch tensor out), so that every step runs on all host threads.  This is the form timed
    as the CPU baseline; tests check it against the numpy functions above.

    vLLM: awq_triton.py:54-101 (unpack order, (q - z) * s), awq.py:276-283 (call site).
    """
    import torch

    shifts = torch.tensor([4 * int(r) for r in AWQ_REVERSE], dtype=torch.int32)

    def unpack(t):
        r, c = t.shape
        return ((t.unsqueeze(-1) >> shifts) & 0xF).reshape(r, c * PACK)

    q = unpack(qweight)
    z = unpack(qzeros).repeat_interleave(group, dim=0)
    w = (q - z).to(torch.float32) * scales.to(torch.float32).repeat_interleave(group, dim=0)
    return x.to(torch.float32) @ w


def pack_kmajor(qweight, group: int = 128) -> np.ndarray:
    """The K-major load-time copy of ``qweight`` that ``awq_b200_repack_kmajor`` produces, as
    bytes: tiles of 256 output columns x one group of 128 k, column slab outermost, group inside;
    row r of a tile is column 256 * slab + r, byte b of the row holds k = 2 b (low nibble) and
    k = 2 b + 1 (high nibble) of the group; columns past N are zero.

    The layout is this repository's own (the reference stack's counterpart is the Marlin repack,
    awq_marlin.py:491-499, a different layout); the values it permutes are those of
    ``unpack_awq`` (awq_triton.py:54-67), which is what pins it.
    """
    q = unpack_awq(qweight)
    k, n = q.shape
    assert group == 128 and k % 128 == 0
    npad = -(-n // 256) * 256
    qp = np.zeros((k, npad), dtype=np.uint8)
    qp[:, :n] = q
    t = qp.reshape(k // 128, 128, npad // 256, 256).transpose(2, 0, 3, 1)  # slab, group, row, k
    return np.ascontiguousarray((t[..., 0::2] | (t[..., 1::2] << 4)).astype(np.uint8)).reshape(-1)


def awq_gemm_fixed_point_model(x, qweight, scales, qzeros, group: int = 128) -> np.ndarray:
    """Model of the arithmetic of this repository's K-major decode kernel (not a restatement of
    the reference): every token is rewritten as 24-bit fixed point X = rint(x * 2^22 / amax), the
    per-group products sum_k q * X are exact integers, and only the fold s * (sum - z * sum_k X)
    runs in fp32 before the result is scaled back by amax / 2^22.  Tests use it to bound what the
    fixed-point step may cost against the fp32 reference (it is below fp16's own rounding)."""
    x = np.asarray(x).astype(np.float32)
    q = unpack_awq(np.asarray(qweight)).astype(np.int64)          # [K, N]
    z = unpack_awq(np.asarray(qzeros)).astype(np.float32)         # [K/G, N]
    s = np.asarray(scales).astype(np.float32)                     # [K/G, N]
    m, k = x.shape
    n = q.shape[1]
    amax = np.abs(x).max(axis=1)
    inv = np.where(amax > 0, np.float32(4194304.0) / np.maximum(amax, np.float32(1e-30)), 0.0)
    xi = np.rint(x * inv[:, None].astype(np.float32)).astype(np.int64)      # |X| <= 2^22
    out = np.zeros((m, n), dtype=np.float32)
    for g in range(k // group):
        rows = slice(g * group, (g + 1) * group)
        v = (xi[:, rows] @ q[rows]).astype(np.float32)            # exact below 2^24 * 15 * 128 ...
        sx = xi[:, rows].sum(axis=1).astype(np.float32)
        out += s[g][None, :] * (v - z[g][None, :] * sx[:, None])
    return out * (amax / np.float32(4194304.0))[:, None].astype(np.float32)


def awq_to_wna16_qweight(qweight) -> np.ndarray:
    """AWQ qweight int32 [K, N/8] -> the "standard" layout of vLLM's MoE WNA16 method:
    uint8 [N, K/2], byte (n, j) = nibble(k=2j) | nibble(k=2j+1) << 4
    (vLLM: model_executor/layers/quantization/moe_wna16.py:389-425, tensor_type "qweight")."""
    q = unpack_awq(qweight)                       # [K, N] nibbles in column order
    t = np.ascontiguousarray(q.T)                 # [N, K]
    return (t[:, 0::2] | (t[:, 1::2] << 4)).astype(np.uint8)


def awq_to_wna16_qzeros(qzeros) -> np.ndarray:
    """AWQ qzeros int32 [K/G, N/8] -> uint8 [N/2, K/G], byte (i, g) = zero(n=2i) |
    zero(n=2i+1) << 4 (same converter, tensor_type "qzeros")."""
    z = unpack_awq(qzeros)                        # [K/G, N]
    t = np.ascontiguousarray(z.T)                 # [N, K/G]
    return (t[0::2, :] | (t[1::2, :] << 4)).astype(np.uint8)


def wna16_to_awq_qweight(w_u8) -> np.ndarray:
    """Inverse of awq_to_wna16_qweight: uint8 [N, K/2] -> int32 [K, N/8]."""
    w = np.asarray(w_u8, dtype=np.uint8)
    n, half = w.shape
    t = np.empty((n, half * 2), dtype=np.uint8)
    t[:, 0::2] = w & 0xF
    t[:, 1::2] = w >> 4
    return pack_awq(np.ascontiguousarray(t.T))


def wna16_to_awq_qzeros(z_u8) -> np.ndarray:
    """Inverse of awq_to_wna16_qzeros: uint8 [N/2, K/G] -> int32 [K/G, N/8]."""
    z = np.asarray(z_u8, dtype=np.uint8)
    half, groups = z.shape
    t = np.empty((half * 2, groups), dtype=np.uint8)
    t[0::2, :] = z & 0xF
    t[1::2, :] = z >> 4
    return pack_awq(np.ascontiguousarray(t.T))


def awq_linear(x, qweight, scales, qzeros, bias=None, group: int = 128) -> np.ndarray:
    """AWQLinearMethod.apply: fp16 output, optional bias added after the product.

    vLLM: awq.py:262-286.
    """
    y = awq_gemm_fp32(x, qweight, scales, qzeros, group)
    if bias is not None:
        y = y + np.asarray(bias).astype(np.float32)
    return y.astype(np.float16)


# --------------------------------------------------------------------------- MoE routing


def topk_softmax(gating: np.ndarray, topk: int, renormalize: bool):
    """softmax over experts -> top-k (ties: lower expert index first) -> optional renormalise.

    Returns (weights f32 [T,k], ids i32 [T,k], token_expert_indices i32 [T,k]) where
    token_expert_indices[t, j] = j * T + t.
    vLLM: model_executor/layers/fused_moe/router/fused_topk_router.py:17-33,69-113.
    """
    g = np.asarray(gating).astype(np.float32)
    t, e = g.shape
    m = g.max(axis=1, keepdims=True)
    p = np.exp(g - m)
    p = p / p.sum(axis=1, keepdims=True)
    # Descending, lower index first on ties.  The order is taken from the logits: softmax is
    # monotonic, so this is the order of the exact probabilities, and it cannot be disturbed by
    # two close logits rounding to the same fp32 probability.
    order = np.argsort(-g, axis=1, kind="stable")[:, :topk]
    w = np.take_along_axis(p, order, axis=1).astype(np.float32)
    if renormalize:
        w = w / w.sum(axis=1, keepdims=True)
    tok = (np.arange(topk, dtype=np.int32)[None, :] * t + np.arange(t, dtype=np.int32)[:, None])
    return w.astype(np.float32), order.astype(np.int32), tok.astype(np.int32)


def sorted_ids_capacity(numel: int, num_experts: int, block: int) -> int:
    """Length of ``sorted_token_ids``.  vLLM: fused_moe/moe_align_block_size.py:74-80."""
    cap = numel + num_experts * (block - 1)
    if numel < num_experts:
        cap = min(numel * block, cap)
    return cap


def moe_align_block_size(topk_ids: np.ndarray, block: int, num_experts: int, expert_map=None):
    """Stable counting sort of the flat (token*topk + slot) indices by expert; each expert's
    run is padded to a multiple of ``block`` with the sentinel ``numel``.

    Returns (sorted_ids i32 [capacity], expert_ids i32 [ceil(capacity/block)],
    num_tokens_post_pad i32 [1]).  Entries of ``sorted_ids`` past ``num_tokens_post_pad`` hold
    the sentinel; entries of ``expert_ids`` past the used blocks hold -1 (the upstream op
    leaves those unspecified, a fixed value is used so the comparison can be exact).
    With ``expert_map`` (global -> local id, -1 = not on this rank) entries routed to absent
    experts are dropped and ``expert_ids`` holds local ids
    (``ignore_invalid_experts=True`` behaviour).
    vLLM: fused_moe/moe_align_block_size.py:19-103 (semantics and the worked example).
    """
    ids = np.asarray(topk_ids).reshape(-1).astype(np.int64)
    numel = ids.size
    cap = sorted_ids_capacity(numel, num_experts, block)
    nblk = -(-cap // block)
    sorted_ids = np.full(cap, numel, dtype=np.int32)
    expert_ids = np.full(nblk, -1, dtype=np.int32)
    pos = 0
    for e in range(num_experts):
        if expert_map is not None and int(expert_map[e]) < 0:
            continue
        idx = np.nonzero(ids == e)[0]  # ascending flat index = stable order
        n = idx.size
        if n == 0:
            continue
        padded = -(-n // block) * block
        sorted_ids[pos:pos + n] = idx
        local = e if expert_map is None else int(expert_map[e])
        expert_ids[pos // block:(pos + padded) // block] = local
        pos += padded
    return sorted_ids, expert_ids, np.array([pos], dtype=np.int32)


def silu_and_mul(gate_up: np.ndarray) -> np.ndarray:
    """silu(x[:, :I]) * x[:, I:].  vLLM: fused_moe.py:1825-1827 (apply_moe_activation SILU)."""
    x = np.asarray(gate_up).astype(np.float32)
    i = x.shape[1] // 2
    g, u = x[:, :i], x[:, i:]
    return g / (1.0 + np.exp(-g)) * u


def fused_experts_fp32(x, w13_q, w13_s, w13_z, w2_q, w2_s, w2_z, topk_weights, topk_ids,
                       group: int = 128, round_intermediate: bool = True) -> np.ndarray:
    """AWQ fused-MoE layer in fp32: per (token, slot) gate_up GEMM -> silu*mul -> down GEMM ->
    times routed weight -> sum over the k slots.

    Weights are stacked AWQ tensors: w13_q i32 [E, H, 2I/8], w13_s f16 [E, H/G, 2I],
    w13_z i32 [E, H/G, 2I/8]; w2_q i32 [E, I, H/8], w2_s f16 [E, I/G, H], w2_z i32 [E, I/G, H/8]
    (vLLM: model_executor/layers/quantization/awq_marlin.py:549-623).
    ``round_intermediate`` rounds the activation between the two GEMMs to fp16, as the
    fp16 intermediate caches of fused_experts_impl do (vLLM: fused_moe.py:1751-1767,
    1801-1867).
    """
    x = np.asarray(x).astype(np.float32)
    t, h = x.shape
    ids = np.asarray(topk_ids)
    wts = np.asarray(topk_weights).astype(np.float32)
    out = np.zeros((t, h), dtype=np.float32)
    for e in np.unique(ids):
        e = int(e)
        tok, slot = np.nonzero(ids == e)
        w13 = dequantize_fp32(w13_q[e], w13_s[e], w13_z[e], group)
        w2 = dequantize_fp32(w2_q[e], w2_s[e], w2_z[e], group)
        a = silu_and_mul(x[tok] @ w13)
        if round_intermediate:
            a = a.astype(np.float16).astype(np.float32)
        y = a @ w2
        np.add.at(out, tok, y * wts[tok, slot][:, None])
    return out


# --------------------------------------------------------------------------- tolerances


def rel_err(y: np.ndarray, ref: np.ndarray) -> float:
    """max |y - ref| / max |ref| -- the "max relative error" used for fp16 outputs."""
    y = np.asarray(y).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    denom = float(np.abs(ref).max()) if ref.size else 1.0
    return float(np.abs(y - ref).max() / (denom if denom > 0 else 1.0)) if ref.size else 0.0


def elementwise_ok(y: np.ndarray, ref: np.ndarray, tol: float = 1e-2) -> bool:
    """|y - ref| <= tol * |ref| + tol * rms(ref) for every element."""
    y = np.asarray(y).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    if ref.size == 0:
        return True
    rms = float(np.sqrt(np.mean(ref * ref)))
    return bool(np.all(np.abs(y - ref) <= tol * np.abs(ref) + tol * rms))
