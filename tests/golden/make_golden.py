"""Generate the golden vectors in this directory from vLLM's own code (run where the vLLM
wheel is installed; no GPU needed):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py

What is produced (``awq_golden.npz``):
  * packed words made by vLLM's pure-Python packer ``quant_utils.awq_pack`` from known nibbles,
  * the fp16 dequantised matrix returned by vLLM's Triton ``awq_dequantize_triton`` and the
    fp16 product returned by ``awq_gemm_triton``, both executed by the Triton CPU interpreter,
  * the worked example of the ``moe_align_block_size`` docstring (transcribed, 1-based expert
    ids made 0-based).
None of the repository's own code is involved, so the vectors pin the oracle independently.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

from vllm.model_executor.layers.quantization.awq_triton import (
    awq_dequantize_triton,
    awq_gemm_triton,
)
from vllm.model_executor.layers.quantization.utils.quant_utils import awq_pack

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [
    # name, M, K, N, group
    ("tiny", 3, 128, 8, 128),
    ("ragged_m", 5, 256, 64, 128),
    ("two_groups", 16, 256, 128, 128),
    ("wide", 1, 384, 256, 128),
    ("g64", 7, 256, 64, 64),
]


def main() -> None:
    out = {}
    gen = torch.Generator().manual_seed(20251125)
    for name, m, k, n, g in CASES:
        q = torch.randint(0, 16, (k, n), dtype=torch.int32, generator=gen)
        z = torch.randint(0, 16, (k // g, n), dtype=torch.int32, generator=gen)
        s = (0.002 + 0.018 * torch.rand(k // g, n, generator=gen)).half()
        x = torch.randn(m, k, generator=gen).half()
        qweight = awq_pack(q, 4, k, n)
        qzeros = awq_pack(z, 4, k // g, n)
        w = awq_dequantize_triton(qweight, s, qzeros)
        y = awq_gemm_triton(x, qweight, s, qzeros, split_k_iters=1)
        out[f"{name}.nibbles"] = q.numpy().astype(np.uint8)
        out[f"{name}.zero_nibbles"] = z.numpy().astype(np.uint8)
        out[f"{name}.qweight"] = qweight.numpy()
        out[f"{name}.qzeros"] = qzeros.numpy()
        out[f"{name}.scales"] = s.numpy()
        out[f"{name}.x"] = x.numpy()
        out[f"{name}.group"] = np.array([g], dtype=np.int32)
        out[f"{name}.w_fp16"] = w.numpy()
        out[f"{name}.y_fp16_triton"] = y.numpy()
    # known-answer word: columns 0..7 hold nibbles 0..7
    kw = awq_pack(torch.arange(8, dtype=torch.int32).reshape(1, 8), 4, 1, 8)
    out["known_word"] = kw.numpy()
    # moe_align_block_size docstring example (expert ids 1..4 in the prose -> 0..3 here)
    out["align.topk_ids"] = np.array([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=np.int32) - 1
    out["align.block"] = np.array([4], dtype=np.int32)
    out["align.num_experts"] = np.array([4], dtype=np.int32)
    out["align.sorted_ids"] = np.array(
        [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12], dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "awq_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "awq_golden.npz"), len(out), "arrays", file=sys.stderr)


if __name__ == "__main__":
    main()
