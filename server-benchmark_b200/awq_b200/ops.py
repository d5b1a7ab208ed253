"""Operator-level API: same names, argument order and meaning as the vLLM ops the
cloudrift-ai/server-benchmark harness exercises (paths are inside the ``vllm`` package):

  awq_gemm(input, qweight, scales, qzeros, split_k_iters)      _custom_ops.py:576-587
  awq_dequantize(qweight, scales, zeros, split_k_iters, thx, thy)   _custom_ops.py:542-556
  fused_topk(hidden_states, gating_output, topk, renormalize, ...)
                                        model_executor/layers/fused_moe/router/fused_topk_router.py:69-113
  moe_align_block_size(topk_ids, block_size, num_experts, expert_map, ...)
                                        model_executor/layers/fused_moe/moe_align_block_size.py:11-103
  fused_experts(hidden_states, w1, w2, topk_weights, topk_ids, ...)
                                        model_executor/layers/fused_moe/fused_moe.py:1587-1631

Every function launches hand-written sm_100a kernels through the C ABI on the current CUDA
stream; nothing here computes on the CPU and nothing synchronises.
"""
from __future__ import annotations

import torch

from . import _lib

PACK_FACTOR = 8
MOE_DIRECT_MAX_PAIRS = 64     # pairs up to which fused_experts goes direct (the limit of the C ABI,
                              # AWQ_B200_MOE_DIRECT_MAX_PAIRS; measured on the Qwen3-30B-A3B layer:
                              # 25 / 33 / 42 / 67 us direct against 30 / 35 / 46 / 74 us through the
                              # permutation at 1 / 2 / 4 / 8 tokens)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require(t: torch.Tensor, name: str, dtype, ndim: int | None = None) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on a CUDA device (there is no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must have {ndim} dimensions, got {t.dim()}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _awq_dims(qweight, scales, qzeros, kmajor: bool = False):
    _require(qweight, "qweight", torch.int32, 2)
    _require(scales, "scales", torch.float16, 2)
    _require(qzeros, "qzeros", torch.int32, 2)
    k, words = qweight.shape
    if kmajor:
        # output of awq_repack_kmajor: [K, ceil(N / 256) * 256 / 8], the true N is that of scales
        n = scales.shape[1]
        if n % PACK_FACTOR or words != -(-n // 256) * 256 // PACK_FACTOR:
            raise ValueError("qweight is not the k-major copy of a matrix with scales' width")
        words = n // PACK_FACTOR
    n = words * PACK_FACTOR
    groups = scales.shape[0]
    if groups == 0 or k == 0 or k % groups != 0:
        raise ValueError(f"K={k} is not a multiple of the number of groups {groups}")
    if tuple(scales.shape) != (groups, n):
        raise ValueError(f"scales must be [{groups}, {n}], got {tuple(scales.shape)}")
    if tuple(qzeros.shape) != (groups, words):
        raise ValueError(f"qzeros must be [{groups}, {words}], got {tuple(qzeros.shape)}")
    return k, n, k // groups


_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_retired: list[torch.Tensor] = []   # outgrown buffers: CUDA graphs captured earlier still use them
_MIN_WORKSPACE = 8 << 20            # covers every dense kernel's scratch need


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor | None:
    """Scratch owned by the torch caching allocator, one buffer per (device, stream).

    A buffer is replaced only when a call needs more than it holds; the old one is kept alive
    (a CUDA graph captured earlier has its address baked in).  Growing while the stream is
    being captured would put the new buffer into the graph's private pool, so that raises:
    size the scratch beforehand with ``reserve_workspace``."""
    if nbytes == 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(
                    f"the scratch buffer of this stream ({ws.numel()} bytes) would have to grow to "
                    f"{nbytes} bytes during stream capture; call "
                    "awq_b200.reserve_workspace(nbytes) on this stream before capturing")
            _retired.append(ws)
        ws = torch.empty(max(nbytes, _MIN_WORKSPACE), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def reserve_workspace(nbytes: int, device: torch.device | str | None = None) -> None:
    """Make the current stream's scratch buffer at least ``nbytes`` large (load-time call, before
    any CUDA-graph capture).  ``moe_workspace_bytes`` gives the need of the fused-MoE layer for a
    token count; the dense kernels never need more than the default."""
    dev = torch.device(device) if device is not None else torch.device("cuda",
                                                                      torch.cuda.current_device())
    _workspace(dev, int(nbytes))


def moe_workspace_bytes(tokens: int, topk: int, num_experts: int, hidden: int,
                        intermediate: int) -> int:
    """Scratch bytes ``fused_experts`` needs for up to ``tokens`` tokens (num_experts: the global
    expert count the routing is done over)."""
    return int(_lib.load().awq_b200_moe_workspace_bytes(tokens, topk, num_experts, hidden,
                                                        intermediate))


def awq_dequantize(qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                   split_k_iters: int = 0, thx: int = 0, thy: int = 0) -> torch.Tensor:
    """W fp16 [K, N] = (q - z) * s.  ``split_k_iters``, ``thx``, ``thy`` are accepted for
    signature compatibility (callers pass 0, 0, 0: quantization/awq.py:280) and ignored."""
    k, n, group = _awq_dims(qweight, scales, zeros)
    out = torch.empty((k, n), dtype=scales.dtype, device=qweight.device)
    rc = _lib.load().awq_b200_dequantize(qweight.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                         out.data_ptr(), k, n, group, _stream())
    _lib.check("awq_b200_dequantize", rc)
    return out


def awq_gemm(input: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
             qzeros: torch.Tensor, split_k_iters: int = 8, *, bias: torch.Tensor | None = None,
             kernel: int = _lib.KERNEL_AUTO, out: torch.Tensor | None = None) -> torch.Tensor:
    """y fp16 [M, N] = input [M, K] @ dequant(qweight), fp32 accumulation.

    ``split_k_iters`` is accepted and ignored (the split along K is chosen from the shape and
    the SM count).  ``bias``, ``kernel`` and ``out`` (a contiguous fp16 [M, N] tensor to write
    into, e.g. a view of a peer-mapped buffer) are keyword-only extensions.
    """
    k, n, group = _awq_dims(qweight, scales, qzeros, kmajor=kernel == _lib.KERNEL_Q8)
    _require(input, "input", torch.float16, 2)
    if input.shape[1] != k:
        raise ValueError(f"input has K={input.shape[1]}, qweight has K={k}")
    if bias is not None:
        _require(bias, "bias", torch.float16, 1)
        if bias.shape[0] != n:
            raise ValueError(f"bias must have {n} elements")
    m = input.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float16, device=input.device)
    else:
        _require(out, "out", torch.float16, 2)
        if out.shape != (m, n):
            raise ValueError(f"out must be [{m}, {n}]")
    if m == 0:
        return out
    lib = _lib.load()
    need = lib.awq_b200_gemm_workspace_bytes(m, n, k, group, kernel)
    ws = _workspace(input.device, need)
    rc = lib.awq_b200_gemm(input.data_ptr(), qweight.data_ptr(), scales.data_ptr(),
                           qzeros.data_ptr(), bias.data_ptr() if bias is not None else None,
                           out.data_ptr(), m, n, k, group, kernel,
                           ws.data_ptr() if ws is not None else None,
                           ws.numel() if ws is not None else 0, _stream())
    _lib.check("awq_b200_gemm", rc)
    return out


def awq_repack(qweight: torch.Tensor) -> torch.Tensor:
    """Decode-layout copy of ``qweight`` for ``awq_gemm(..., kernel=KERNEL_STREAM_RP)``.

    The copy holds, for every four rows k..k+3 and packed word column c, the four 32-bit
    words the streaming kernel otherwise builds with byte permutes: the low and the high
    halfwords of the row pairs (k, k+1) and (k+2, k+3).  It is returned with the shape of
    ``qweight`` ([K, N/8] int32; memory order [K/4, N/8, 4]) so that it can be passed where
    ``qweight`` goes; no other kernel understands it.  A stacked expert tensor [E, K, N/8] is
    repacked expert by expert (for ``fused_experts(..., w1_decode=, w2_decode=)``).  Load-time counterpart of the Marlin
    repack in vllm/model_executor/layers/quantization/awq_marlin.py:491-499.
    """
    _require(qweight, "qweight", torch.int32)
    if qweight.dim() not in (2, 3):
        raise ValueError("qweight must be [K, N/8] or stacked [E, K, N/8]")
    k, words = qweight.shape[-2:]
    if k % 4:
        raise ValueError("K must be a multiple of 4")
    out = torch.empty_like(qweight)
    if qweight.numel():
        # stacked experts: K % 4 == 0, so no row quad crosses an expert and the stack repacks
        # as one [E * K, N/8] matrix
        rc = _lib.load().awq_b200_repack_qweight(qweight.data_ptr(), out.data_ptr(),
                                                 qweight.numel() // words, words * 8, _stream())
        _lib.check("awq_b200_repack_qweight", rc)
        # Load-time operation: finish it here.  The GEMM kernels prefetch weights before they
        # wait for the kernel ahead of them in the stream, so a copy still being written must
        # not be handed to them.
        torch.cuda.current_stream().synchronize()
    return out


def awq_repack_kmajor(qweight: torch.Tensor) -> torch.Tensor:
    """K-major copy of ``qweight`` for ``awq_gemm(..., kernel=KERNEL_Q8)`` (up to 32 tokens).

    The same nibbles running along K, in 16 KB tiles of 256 output columns x one quantisation
    group, column slabs outermost (include/awq_b200.h, awq_b200_repack_kmajor).  Returned as
    int32 [K, ceil(N / 256) * 256 / 8]: the size of ``qweight`` when N is a multiple of 256.
    K must be a multiple of 128.  Load-time counterpart of the Marlin repack in
    vllm/model_executor/layers/quantization/awq_marlin.py:491-499.
    """
    _require(qweight, "qweight", torch.int32, 2)
    k, words = qweight.shape
    n = words * PACK_FACTOR
    lib = _lib.load()
    nbytes = int(lib.awq_b200_repack_kmajor_bytes(k, n))
    if nbytes == 0:
        raise ValueError("K must be a positive multiple of 128")
    out = torch.empty((k, nbytes // (4 * k)), dtype=torch.int32, device=qweight.device)
    rc = lib.awq_b200_repack_kmajor(qweight.data_ptr(), out.data_ptr(), k, n, _stream())
    _lib.check("awq_b200_repack_kmajor", rc)
    # load-time operation: the GEMM kernels prefetch weights before they wait for the kernel
    # ahead of them in the stream, so the copy must be complete before it is handed to them
    torch.cuda.current_stream().synchronize()
    return out


def wna16_to_awq(w: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                 group_size: int = 128):
    """Stacked expert tensors in the byte layout of vLLM's MoE WNA16 method (w uint8 [E, N, K/2],
    scales fp16 [E, N, K/G], zeros uint8 [E, N/2, K/G]; moe_wna16.py:252-324) -> the AWQ
    checkpoint layout ``fused_experts`` takes: (qweight i32 [E, K, N/8], scales f16 [E, K/G, N],
    qzeros i32 [E, K/G, N/8]).  Load time; bit-exact inverse of vLLM's converter
    (moe_wna16.py:389-425)."""
    _require(w, "w", torch.uint8, 3)
    _require(scales, "scales", torch.float16, 3)
    _require(zeros, "zeros", torch.uint8, 3)
    e, n, half = w.shape
    k = 2 * half
    if n % PACK_FACTOR != 0 or k % group_size != 0:
        raise ValueError("N must be a multiple of 8 and K a multiple of the group size")
    g = k // group_size
    if scales.shape != (e, n, g) or zeros.shape != (e, n // 2, g):
        raise ValueError("scales / zeros shapes do not match w and the group size")
    qweight = torch.empty((e, k, n // PACK_FACTOR), dtype=torch.int32, device=w.device)
    qzeros = torch.empty((e, g, n // PACK_FACTOR), dtype=torch.int32, device=w.device)
    s_out = torch.empty((e, g, n), dtype=torch.float16, device=w.device)
    rc = _lib.load().awq_b200_wna16_to_awq(w.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                           qweight.data_ptr(), s_out.data_ptr(),
                                           qzeros.data_ptr(), e, n, k, group_size, _stream())
    _lib.check("awq_b200_wna16_to_awq", rc)
    return qweight, s_out, qzeros


# ------------------------------------------------------------------------------- MoE


def fused_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, topk: int,
               renormalize: bool, indices_type: torch.dtype | None = None,
               scoring_func: str = "softmax"):
    """softmax -> top-k -> optional renormalise.  Returns (topk_weights f32 [T,k],
    topk_ids i32 [T,k], token_expert_indices i32 [T,k])."""
    if scoring_func != "softmax":
        raise ValueError(f"Unsupported scoring function: {scoring_func}")
    if hidden_states.shape[0] != gating_output.shape[0]:
        raise ValueError("Number of tokens mismatch")
    if indices_type not in (None, torch.int32):
        raise ValueError("indices_type must be torch.int32")
    if gating_output.dtype == torch.float32:
        gd = 0
    elif gating_output.dtype == torch.float16:
        gd = 1
    else:
        raise ValueError("gating_output must be float32 or float16")
    _require(gating_output, "gating_output", gating_output.dtype, 2)
    t, e = gating_output.shape
    dev = gating_output.device
    w = torch.empty((t, topk), dtype=torch.float32, device=dev)
    ids = torch.empty((t, topk), dtype=torch.int32, device=dev)
    tok = torch.empty((t, topk), dtype=torch.int32, device=dev)
    if t > 0:
        rc = _lib.load().awq_b200_topk_softmax(gating_output.data_ptr(), gd, t, e, topk,
                                               int(bool(renormalize)), w.data_ptr(),
                                               ids.data_ptr(), tok.data_ptr(), _stream())
        _lib.check("awq_b200_topk_softmax", rc)
    return w, ids, tok


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int,
                         expert_map: torch.Tensor | None = None, pad_sorted_ids: bool = False,
                         ignore_invalid_experts: bool = False):
    """Token -> expert permutation.  Returns (sorted_token_ids, expert_ids,
    num_tokens_post_padded), all int32 on the device."""
    _require(topk_ids, "topk_ids", torch.int32, 2)
    lib = _lib.load()
    t, k = topk_ids.shape
    cap = int(lib.awq_b200_moe_sorted_capacity(t * k, num_experts, block_size))
    if pad_sorted_ids:
        cap = -(-cap // block_size) * block_size
    dev = topk_ids.device
    sorted_ids = torch.empty((cap,), dtype=torch.int32, device=dev)
    nblk = -(-cap // block_size) if cap > 0 else 0
    expert_ids = torch.empty((nblk,), dtype=torch.int32, device=dev)
    num_post = torch.empty((1,), dtype=torch.int32, device=dev)
    emap = None
    if expert_map is not None and ignore_invalid_experts:
        _require(expert_map, "expert_map", torch.int32, 1)
        emap = expert_map
    rc = lib.awq_b200_moe_align_block_size(topk_ids.data_ptr(), t, k, num_experts, block_size,
                                           emap.data_ptr() if emap is not None else None,
                                           sorted_ids.data_ptr(), cap, expert_ids.data_ptr(),
                                           num_post.data_ptr(), _stream())
    _lib.check("awq_b200_moe_align_block_size", rc)
    if expert_map is not None and not ignore_invalid_experts:
        # same post-processing as the reference wrapper (moe_align_block_size.py:100-101);
        # unused trailing blocks stay -1
        used = expert_ids >= 0
        expert_ids = torch.where(used, expert_map[expert_ids.clamp(min=0).long()].to(torch.int32),
                                 expert_ids)
    return sorted_ids, expert_ids, num_post


def fused_experts(hidden_states: torch.Tensor, w1, w2, topk_weights: torch.Tensor,
                  topk_ids: torch.Tensor, inplace: bool = False, activation: str = "silu",
                  apply_router_weight_on_input: bool = False, global_num_experts: int = -1,
                  expert_map: torch.Tensor | None = None, group_size: int = 128,
                  w1_decode: torch.Tensor | None = None,
                  w2_decode: torch.Tensor | None = None, quant_config=None) -> torch.Tensor:
    """AWQ fused-MoE experts.  ``w1`` and ``w2`` are (qweight, scales, qzeros) triples of the
    stacked AWQ tensors: w1 = (i32 [E,H,2I/8], f16 [E,H/G,2I], i32 [E,H/G,2I/8]),
    w2 = (i32 [E,I,H/8], f16 [E,I/G,H], i32 [E,I/G,H/8]).  Returns fp16 [T, H].

    The form of vLLM's ``fused_experts`` (fused_moe/fused_moe.py:1587-1599) is accepted too:
    ``w1`` / ``w2`` the two stacked qweight tensors and ``quant_config`` an object carrying
    ``w1_scale``, ``w2_scale``, ``w1_zp``, ``w2_zp`` (a ``FusedMoEQuantConfig``, e.g. from
    ``int4_w4a16_moe_quant_config``); its ``block_shape[1]``, when set, is the group size.

    ``w1_decode`` / ``w2_decode`` (both or neither): ``awq_repack`` of the two stacked qweights,
    made once at load time.  Batches small enough for the weight-streaming expert kernels
    (``awq_b200_moe_block_size`` 8 or 16, group 128) then read those copies; larger batches
    use ``w1`` / ``w2`` as always."""
    if activation != "silu":
        raise ValueError("only the silu activation is implemented")
    if apply_router_weight_on_input:
        raise ValueError("apply_router_weight_on_input is not implemented")
    if quant_config is not None:
        if not (torch.is_tensor(w1) and torch.is_tensor(w2)):
            raise ValueError("with quant_config, w1 and w2 are the stacked qweight tensors")
        w1 = (w1, quant_config.w1_scale, quant_config.w1_zp)
        w2 = (w2, quant_config.w2_scale, quant_config.w2_zp)
        if w1[1] is None or w1[2] is None or w2[1] is None or w2[2] is None:
            raise ValueError("quant_config must carry w1_scale, w2_scale, w1_zp and w2_zp")
        shape = getattr(quant_config, "block_shape", None)
        if shape is not None and len(shape) == 2 and shape[1]:
            group_size = int(shape[1])
    elif torch.is_tensor(w1) or torch.is_tensor(w2):
        raise ValueError("w1 and w2 are (qweight, scales, qzeros) triples, or tensors together "
                         "with quant_config")
    w13_q, w13_s, w13_z = w1
    w2_q, w2_s, w2_z = w2
    _require(hidden_states, "hidden_states", torch.float16, 2)
    _require(w13_q, "w1.qweight", torch.int32, 3)
    _require(w13_s, "w1.scales", torch.float16, 3)
    _require(w13_z, "w1.qzeros", torch.int32, 3)
    _require(w2_q, "w2.qweight", torch.int32, 3)
    _require(w2_s, "w2.scales", torch.float16, 3)
    _require(w2_z, "w2.qzeros", torch.int32, 3)
    _require(topk_weights, "topk_weights", torch.float32, 2)
    _require(topk_ids, "topk_ids", torch.int32, 2)
    t, h = hidden_states.shape
    e = w13_q.shape[0]
    inter = w2_q.shape[1]
    topk = topk_ids.shape[1]
    g = group_size
    if w13_q.shape != (e, h, 2 * inter // 8) or w2_q.shape != (e, inter, h // 8):
        raise ValueError("expert weight shapes do not match hidden/intermediate sizes")
    if w13_s.shape != (e, h // g, 2 * inter) or w13_z.shape != (e, h // g, 2 * inter // 8):
        raise ValueError("w1 scales/zeros shapes do not match group size")
    if w2_s.shape != (e, inter // g, h) or w2_z.shape != (e, inter // g, h // 8):
        raise ValueError("w2 scales/zeros shapes do not match group size")
    if topk_weights.shape != (t, topk):
        raise ValueError("topk_weights / topk_ids shape mismatch")
    if global_num_experts not in (-1, e) and expert_map is None:
        raise ValueError("global_num_experts differs from the stacked expert count")
    if (w1_decode is None) != (w2_decode is None):
        raise ValueError("w1_decode and w2_decode go together")
    if w1_decode is not None:
        _require(w1_decode, "w1_decode", torch.int32, 3)
        _require(w2_decode, "w2_decode", torch.int32, 3)
        if w1_decode.shape != w13_q.shape or w2_decode.shape != w2_q.shape:
            raise ValueError("decode-layout copies must have the shapes of the qweights")
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    if t == 0:
        return out
    lib = _lib.load()
    n_global = e if global_num_experts == -1 else global_num_experts
    block = lib.awq_b200_moe_block_size(t, topk, n_global, h, inter, g)
    flags = int(expert_map is not None)
    if w1_decode is not None and block in (8, 16) and g == 128:
        w13_q, w2_q = w1_decode, w2_decode
        flags |= 2
    need = lib.awq_b200_moe_workspace_bytes(t, topk, n_global, h, inter)
    ws = _workspace(hidden_states.device, need)
    if (expert_map is None and block == 8 and t * topk <= MOE_DIRECT_MAX_PAIRS
            and t * topk * 8 <= lib.awq_b200_moe_sorted_capacity(t * topk, n_global, 16)):
        # (the last condition: the scratch bound of awq_b200_moe_workspace_bytes covers one 8-row
        # block per pair only while the pairs are few compared with the experts)
        # a handful of pairs: one row block per pair straight from topk_ids, no permutation
        rc = lib.awq_b200_moe_experts(
            hidden_states.data_ptr(), w13_q.data_ptr(), w13_s.data_ptr(), w13_z.data_ptr(),
            w2_q.data_ptr(), w2_s.data_ptr(), w2_z.data_ptr(), topk_weights.data_ptr(),
            None, topk_ids.data_ptr(), None, out.data_ptr(),
            t, topk, e, h, inter, g, block, flags | 4, t * topk * 8,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            _stream())
        _lib.check("awq_b200_moe_experts", rc)
        return out
    sorted_ids, expert_ids, num_post = moe_align_block_size(
        topk_ids, block, n_global, expert_map, ignore_invalid_experts=True)
    rc = lib.awq_b200_moe_experts(
        hidden_states.data_ptr(), w13_q.data_ptr(), w13_s.data_ptr(), w13_z.data_ptr(),
        w2_q.data_ptr(), w2_s.data_ptr(), w2_z.data_ptr(), topk_weights.data_ptr(),
        sorted_ids.data_ptr(), expert_ids.data_ptr(), num_post.data_ptr(), out.data_ptr(),
        t, topk, e, h, inter, g, block, flags, sorted_ids.numel(),
        ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
        _stream())
    _lib.check("awq_b200_moe_experts", rc)
    return out


def fused_moe(hidden_states: torch.Tensor, w1, w2, gating_output: torch.Tensor, topk: int,
              renormalize: bool, inplace: bool = False, group_size: int = 128) -> torch.Tensor:
    """Routing followed by the experts: fused_topk then fused_experts (the historical
    ``fused_moe`` entry point older call sites use)."""
    w, ids, _ = fused_topk(hidden_states, gating_output, topk, renormalize)
    return fused_experts(hidden_states, w1, w2, w, ids, inplace=inplace, group_size=group_size)
