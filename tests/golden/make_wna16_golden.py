"""Golden vectors for the MoE WNA16 weight layout, made by vLLM's own converter (run where the
vLLM wheel is installed; no GPU needed):

    python tests/golden/make_wna16_golden.py

vLLM converts AWQ expert tensors inside the weight loader that
``MoeWNA16Method.get_weight_loader`` returns (moe_wna16.py:387-512).  This script builds that
loader around a stub layer and a capturing inner loader, feeds it AWQ tensors packed by vLLM's
``awq_pack`` and stores what comes out (``wna16_golden.npz``).  None of the repository's own code
is involved."""
import os
import sys
from types import SimpleNamespace
from unittest import mock

import numpy as np
import torch

from vllm.model_executor.layers.quantization import moe_wna16
from vllm.model_executor.layers.quantization.utils.quant_utils import awq_pack

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [("small", 256, 64, 128), ("wide", 128, 256, 128), ("g64", 256, 128, 64)]   # K, N, G


def main() -> None:
    out = {}
    gen = torch.Generator().manual_seed(20251126)
    for name, k, n, g in CASES:
        q = torch.randint(0, 16, (k, n), dtype=torch.int32, generator=gen)
        z = torch.randint(0, 16, (k // g, n), dtype=torch.int32, generator=gen)
        s = (0.002 + 0.018 * torch.rand(k // g, n, generator=gen)).half()
        qweight = awq_pack(q, 4, k, n)
        qzeros = awq_pack(z, 4, k // g, n)
        layer = SimpleNamespace(
            quant_config=SimpleNamespace(has_zp=True, linear_quant_method="awq", weight_bits=4),
            intermediate_size_per_partition=k, group_size_div_factor=1, tp_size=1)
        got = {}

        def inner(param, loaded_weight, weight_name, shard_id, expert_id, return_success=False):
            got[weight_name] = loaded_weight.clone()

        loader = moe_wna16.MoeWNA16Method.get_weight_loader(layer, inner)
        zparam = SimpleNamespace(data=torch.zeros(1, n // 2, k // g, dtype=torch.uint8))
        with mock.patch.object(moe_wna16, "get_tp_group", lambda: SimpleNamespace(device="cpu")), \
                mock.patch.object(moe_wna16, "get_tensor_model_parallel_rank", lambda: 0):
            loader(None, qweight, "w2_qweight", "w2", 0)
            loader(None, s, "w2_scales", "w2", 0)
            loader(zparam, qzeros, "w2_qzeros", "w2", 0)
        out[f"{name}.qweight"] = qweight.numpy()
        out[f"{name}.qzeros"] = qzeros.numpy()
        out[f"{name}.scales"] = s.numpy()
        out[f"{name}.group"] = np.array([g], dtype=np.int32)
        out[f"{name}.wna16_qweight"] = got["w2_qweight"].numpy()
        out[f"{name}.wna16_scales"] = got["w2_scales"].contiguous().numpy()
        out[f"{name}.wna16_qzeros"] = zparam.data[0].numpy()
    np.savez_compressed(os.path.join(HERE, "wna16_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "wna16_golden.npz"), len(out), "arrays", file=sys.stderr)


if __name__ == "__main__":
    main()
