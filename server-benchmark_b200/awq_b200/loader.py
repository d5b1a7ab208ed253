"""AWQ checkpoints (AutoAWQ ``version: gemm`` safetensors) -> the tensors this package's layers
take, without vLLM: per-module ``qweight`` / ``qzeros`` / ``scales`` read by name, the fused
projections of a decoder stacked the way vLLM's parallel linears stack their shards, expert
tensors stacked over experts, and tensor-parallel shards cut on the same boundaries.

Counterparts in the reference stack (paths inside the ``vllm`` package):
  quantization config of a checkpoint     model_executor/layers/quantization/awq.py:87-95
  modules_to_not_convert                  quantization/awq.py:145-169, utils/quant_utils.py
  fused qkv / gate_up shard stacking      model_executor/layers/linear.py (QKVParallelLinear,
                                          MergedColumnParallelLinear weight loaders)
  per-expert names -> w13 / w2 stacks     fused_moe/layer.py make_expert_params_mapping,
                                          quantization/awq_marlin.py:549-623 (parameter shapes)

With the plug-in (``awq_b200.vllm_plugin``) none of this is needed: the plug-in's methods declare
vLLM's own parameters, so vLLM's checkpoint loader fills them.  This module serves hosts that use
``awq_b200.linear`` / ``awq_b200.ops`` directly.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch

PACK_FACTOR = 8
SUFFIXES = ("qweight", "qzeros", "scales")


@dataclass
class AWQCheckpointConfig:
    """The ``quantization_config`` block of config.json (or quant_config.json / quantize_config.json)."""

    weight_bits: int
    group_size: int
    zero_point: bool
    modules_to_not_convert: list[str]

    @classmethod
    def from_dict(cls, cfg: dict) -> "AWQCheckpointConfig":
        method = str(cfg.get("quant_method", "awq")).lower()
        if method != "awq":
            raise ValueError(f"not an AWQ checkpoint: quant_method = {method!r}")

        def first(*keys, default=None):
            for k in keys:
                if k in cfg:
                    return cfg[k]
            if default is None:
                raise ValueError(f"Cannot find any of {list(keys)} in the model's quantization config.")
            return default

        bits = int(first("w_bit", "bits"))
        if bits != 4:
            raise ValueError("Currently, only 4-bit weight quantization is supported for AWQ, "
                             f"but got {bits} bits.")
        return cls(bits, int(first("q_group_size", "group_size")),
                   bool(first("zero_point")),
                   list(first("modules_to_not_convert", default=[]) or []))

    @classmethod
    def from_model_dir(cls, path: str) -> "AWQCheckpointConfig":
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        if "quantization_config" in cfg:
            return cls.from_dict(cfg["quantization_config"])
        for name in ("quant_config.json", "quantize_config.json"):
            p = os.path.join(path, name)
            if os.path.exists(p):
                with open(p) as f:
                    return cls.from_dict(json.load(f))
        raise ValueError("the model directory holds no quantization config")

    def is_skipped(self, prefix: str) -> bool:
        """Substring match, as vLLM applies modules_to_not_convert to AWQ checkpoints."""
        return any(m in prefix for m in self.modules_to_not_convert)


class SafetensorsIndex:
    """Tensor name -> file, over every *.safetensors of a directory (the weight map of
    model.safetensors.index.json when present)."""

    def __init__(self, path: str) -> None:
        from safetensors import safe_open
        self.path = path
        self._open = safe_open
        self.where: dict[str, str] = {}
        index = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                self.where = dict(json.load(f)["weight_map"])
        else:
            for name in sorted(os.listdir(path)):
                if name.endswith(".safetensors"):
                    with safe_open(os.path.join(path, name), framework="pt") as f:
                        for key in f.keys():
                            self.where[key] = name
        if not self.where:
            raise ValueError(f"no safetensors weights under {path}")

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise KeyError(f"tensor {name!r} is not in the checkpoint")
        with self._open(os.path.join(self.path, self.where[name]), framework="pt") as f:
            return f.get_tensor(name)


def load_awq_module(index: SafetensorsIndex, prefix: str):
    """(qweight i32 [K, N/8], scales f16 [K/G, N], qzeros i32 [K/G, N/8]) of one module."""
    qweight = index.get(f"{prefix}.qweight")
    qzeros = index.get(f"{prefix}.qzeros")
    scales = index.get(f"{prefix}.scales")
    if qweight.dtype != torch.int32 or qzeros.dtype != torch.int32:
        raise ValueError(f"{prefix}: qweight / qzeros must be int32")
    k, words = qweight.shape
    groups = scales.shape[0]
    if scales.shape[1] != words * PACK_FACTOR or qzeros.shape != (groups, words) or k % groups:
        raise ValueError(f"{prefix}: qweight {tuple(qweight.shape)}, qzeros {tuple(qzeros.shape)} "
                         f"and scales {tuple(scales.shape)} do not describe one AWQ matrix")
    return qweight, scales.to(torch.float16), qzeros


def fuse_columns(parts):
    """Stack projections that share their input along N (q,k,v -> qkv; gate,up -> gate_up).  Every
    part has N % 8 == 0, so whole packed words are concatenated and no nibble moves."""
    ks = {p[0].shape[0] for p in parts}
    gs = {p[1].shape[0] for p in parts}
    if len(ks) != 1 or len(gs) != 1:
        raise ValueError("fused projections must share K and the group size")
    return (torch.cat([p[0] for p in parts], dim=1).contiguous(),
            torch.cat([p[1] for p in parts], dim=1).contiguous(),
            torch.cat([p[2] for p in parts], dim=1).contiguous())


def load_fused(index: SafetensorsIndex, prefix: str, names: list[str]):
    """e.g. load_fused(idx, "model.layers.0.self_attn", ["q_proj", "k_proj", "v_proj"])."""
    return fuse_columns([load_awq_module(index, f"{prefix}.{n}") for n in names])


def load_experts(index: SafetensorsIndex, prefix: str, num_experts: int,
                 gate: str = "gate_proj", up: str = "up_proj", down: str = "down_proj"):
    """Stacked expert tensors for ``ops.fused_experts``: w1 = (w13_qweight [E, H, 2I/8],
    w13_scales [E, H/G, 2I], w13_qzeros [E, H/G, 2I/8]) with gate before up, and w2 likewise."""
    w13, w2 = [], []
    for e in range(num_experts):
        base = f"{prefix}.{e}"
        w13.append(fuse_columns([load_awq_module(index, f"{base}.{gate}"),
                                 load_awq_module(index, f"{base}.{up}")]))
        w2.append(load_awq_module(index, f"{base}.{down}"))
    stack = lambda items: tuple(torch.stack([it[j] for it in items]).contiguous()  # noqa: E731
                                for j in range(3))
    return stack(w13), stack(w2)


def fused_shard_columns(parts, rank: int, world: int):
    """Tensor-parallel shard of a fused column-parallel projection: every part is cut into
    ``world`` column ranges and rank ``rank`` keeps its range of each, in part order (the layout
    QKVParallelLinear / MergedColumnParallelLinear hold on one rank)."""
    from .tp import shard_columns
    return fuse_columns([shard_columns(*p, rank, world) for p in parts])
