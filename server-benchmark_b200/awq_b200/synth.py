"""Seeded synthetic AWQ tensors with the value distributions the benchmark configurations
name: nibbles uniform in 0..15 (weights and zero points), scales uniform in [0.002, 0.02],
activations ~ N(0, 1) in fp16.  Everything is drawn on the CPU from a torch.Generator so the
same seed gives the same tensors on every machine; callers move them to the GPU.
"""
from __future__ import annotations

import torch

PACK_FACTOR = 8
# nibble p (LSB first) of a packed word holds column AWQ_ORDER[p] of its 8 columns
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)

# (K, N) of the four AWQ linears of one Qwen2.5-72B decoder layer
QWEN25_72B_SHAPES = {
    "qkv": (8192, 10240),
    "o_proj": (8192, 8192),
    "gate_up": (8192, 59136),
    "down": (29568, 8192),
}
SWEEP_M = (1, 4, 16, 64, 256, 1024, 4096)

# Qwen3-30B-A3B MoE layer
QWEN3_MOE = dict(hidden=2048, experts=128, intermediate=768, topk=8)
MOE_TOKENS = (1, 16, 128, 1024, 4096)


def random_packed(rows: int, cols: int, gen: torch.Generator) -> torch.Tensor:
    """int32 [rows, cols/8] whose 8 nibbles per word are independent uniform 0..15 values.
    Drawing the word directly is the same distribution as drawing nibbles and packing them in
    any order, and avoids materialising the unpacked matrix for the large shapes."""
    assert cols % PACK_FACTOR == 0
    w = torch.randint(-(2 ** 31), 2 ** 31, (rows, cols // PACK_FACTOR), dtype=torch.int64,
                      generator=gen)
    return w.to(torch.int32)


def pack_awq(q: torch.Tensor) -> torch.Tensor:
    """[R, C] integer nibbles -> int32 [R, C/8] in AWQ order (for tests that need known nibbles)."""
    r, c = q.shape
    g = q.reshape(r, c // PACK_FACTOR, PACK_FACTOR).to(torch.int64)
    word = torch.zeros((r, c // PACK_FACTOR), dtype=torch.int64)
    for p, col in enumerate(AWQ_ORDER):
        word |= (g[:, :, col] & 0xF) << (4 * p)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


def awq_linear_tensors(k: int, n: int, group: int = 128, seed: int = 0):
    """(qweight i32 [K,N/8], scales f16 [K/G,N], qzeros i32 [K/G,N/8]) on the CPU."""
    gen = torch.Generator().manual_seed(seed)
    qweight = random_packed(k, n, gen)
    qzeros = random_packed(k // group, n, gen)
    scales = (0.002 + 0.018 * torch.rand(k // group, n, generator=gen)).to(torch.float16)
    return qweight, scales, qzeros


def activations(m: int, k: int, seed: int = 0) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed + 1_000_003)
    return torch.randn(m, k, generator=gen).to(torch.float16)


def moe_layer_tensors(experts: int, hidden: int, intermediate: int, group: int = 128,
                      seed: int = 0):
    """Stacked AWQ expert weights: (w13_q, w13_s, w13_z), (w2_q, w2_s, w2_z) on the CPU."""
    gen = torch.Generator().manual_seed(seed + 7)
    e, h, i = experts, hidden, intermediate
    w13_q = random_packed(e * h, 2 * i, gen).reshape(e, h, 2 * i // PACK_FACTOR)
    w13_z = random_packed(e * (h // group), 2 * i, gen).reshape(e, h // group, 2 * i // PACK_FACTOR)
    w13_s = (0.002 + 0.018 * torch.rand(e, h // group, 2 * i, generator=gen)).to(torch.float16)
    w2_q = random_packed(e * i, h, gen).reshape(e, i, h // PACK_FACTOR)
    w2_z = random_packed(e * (i // group), h, gen).reshape(e, i // group, h // PACK_FACTOR)
    w2_s = (0.002 + 0.018 * torch.rand(e, i // group, h, generator=gen)).to(torch.float16)
    return (w13_q, w13_s, w13_z), (w2_q, w2_s, w2_z)


def gating_logits(t: int, experts: int, seed: int = 0) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed + 13)
    return torch.randn(t, experts, generator=gen)
