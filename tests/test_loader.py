"""AWQ safetensors checkpoints read without vLLM (awq_b200.loader): module tensors by name, fused
projections, stacked experts, skipped modules, tensor-parallel shards of fused projections, all
against the oracle's dequantisation of the same tensors."""
import json

import numpy as np
import pytest
import torch

from awq_b200 import loader, synth
from oracle import awq_oracle as O


@pytest.fixture()
def checkpoint(tmp_path):
    from safetensors.torch import save_file
    h, inter, e = 256, 128, 3
    tensors, truth = {}, {}

    def add(prefix, k, n, seed):
        qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=seed)
        for suffix, t in zip(("qweight", "scales", "qzeros"), (qw, s, qz)):
            tensors[f"{prefix}.{suffix}"] = t
        truth[prefix] = O.dequantize_fp32(qw.numpy(), s.numpy(), qz.numpy(), 128)

    attn = "model.layers.0.self_attn"
    add(f"{attn}.q_proj", h, 256, 1), add(f"{attn}.k_proj", h, 64, 2), add(f"{attn}.v_proj", h, 64, 3)
    add(f"{attn}.o_proj", 256, h, 4)
    for i in range(e):
        base = f"model.layers.0.mlp.experts.{i}"
        add(f"{base}.gate_proj", h, inter, 10 + i)
        add(f"{base}.up_proj", h, inter, 20 + i)
        add(f"{base}.down_proj", inter, h, 30 + i)
    tensors["model.layers.0.mlp.gate.weight"] = torch.randn(e, h).half()
    half = dict(list(tensors.items())[: len(tensors) // 2])
    rest = {k: v for k, v in tensors.items() if k not in half}
    save_file(half, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(rest, str(tmp_path / "model-00002-of-00002.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({
        "quantization_config": {"quant_method": "awq", "bits": 4, "group_size": 128,
                                "zero_point": True, "version": "gemm",
                                "modules_to_not_convert": ["mlp.gate"]}}))
    return str(tmp_path), truth, (h, inter, e)


def test_config_and_skipped_modules(checkpoint):
    path, _, _ = checkpoint
    cfg = loader.AWQCheckpointConfig.from_model_dir(path)
    assert (cfg.weight_bits, cfg.group_size, cfg.zero_point) == (4, 128, True)
    assert cfg.is_skipped("model.layers.0.mlp.gate") and not cfg.is_skipped("model.layers.0.mlp.experts.0.gate_proj")
    with pytest.raises(ValueError):
        loader.AWQCheckpointConfig.from_dict({"quant_method": "awq", "bits": 8, "group_size": 128,
                                              "zero_point": True})
    with pytest.raises(ValueError):
        loader.AWQCheckpointConfig.from_dict({"quant_method": "gptq", "bits": 4})
    old_style = loader.AWQCheckpointConfig.from_dict({"w_bit": 4, "q_group_size": 64,
                                                      "zero_point": True})
    assert old_style.group_size == 64


def test_fused_qkv_and_single_module(checkpoint):
    path, truth, _ = checkpoint
    idx = loader.SafetensorsIndex(path)
    attn = "model.layers.0.self_attn"
    qkv = loader.load_fused(idx, attn, ["q_proj", "k_proj", "v_proj"])
    w = O.dequantize_fp32(*[t.numpy() for t in (qkv[0], qkv[1], qkv[2])], 128)
    want = np.concatenate([truth[f"{attn}.{n}"] for n in ("q_proj", "k_proj", "v_proj")], axis=1)
    assert np.array_equal(w, want)
    o = loader.load_awq_module(idx, f"{attn}.o_proj")
    assert np.array_equal(O.dequantize_fp32(o[0].numpy(), o[1].numpy(), o[2].numpy(), 128),
                          truth[f"{attn}.o_proj"])
    with pytest.raises(KeyError):
        loader.load_awq_module(idx, f"{attn}.missing")


def test_stacked_experts(checkpoint):
    path, truth, (h, inter, e) = checkpoint
    idx = loader.SafetensorsIndex(path)
    w1, w2 = loader.load_experts(idx, "model.layers.0.mlp.experts", e)
    assert tuple(w1[0].shape) == (e, h, 2 * inter // 8) and tuple(w1[1].shape) == (e, h // 128, 2 * inter)
    assert tuple(w2[0].shape) == (e, inter, h // 8) and tuple(w2[2].shape) == (e, inter // 128, h // 8)
    for i in range(e):
        base = f"model.layers.0.mlp.experts.{i}"
        w13 = O.dequantize_fp32(w1[0][i].numpy(), w1[1][i].numpy(), w1[2][i].numpy(), 128)
        assert np.array_equal(w13[:, :inter], truth[f"{base}.gate_proj"])     # gate first
        assert np.array_equal(w13[:, inter:], truth[f"{base}.up_proj"])
        assert np.array_equal(O.dequantize_fp32(w2[0][i].numpy(), w2[1][i].numpy(),
                                                w2[2][i].numpy(), 128), truth[f"{base}.down_proj"])


def test_tensor_parallel_shard_of_fused_projection(checkpoint):
    path, truth, _ = checkpoint
    idx = loader.SafetensorsIndex(path)
    attn = "model.layers.0.self_attn"
    parts = [loader.load_awq_module(idx, f"{attn}.{n}") for n in ("q_proj", "k_proj", "v_proj")]
    world = 2
    for rank in range(world):
        sh = loader.fused_shard_columns(parts, rank, world)
        w = O.dequantize_fp32(sh[0].numpy(), sh[1].numpy(), sh[2].numpy(), 128)
        want = np.concatenate([
            truth[f"{attn}.{n}"][:, rank * wdt // world:(rank + 1) * wdt // world]
            for n, wdt in (("q_proj", 256), ("k_proj", 64), ("v_proj", 64))], axis=1)
        assert np.array_equal(w, want)
