"""vLLM plugin: put the sm_100a kernels of this package under an unmodified vLLM.

Two hooks, both installed by ``register()`` (entry point of group ``vllm.general_plugins`` in the
pyproject.toml next to this package; vLLM loads those in the API server, the engine core and
every worker, vllm/plugins/__init__.py:28-82; the function is idempotent, as vLLM requires):

1. **Quantization configs.**  ``"awq"``, ``"awq_marlin"`` and ``"moe_wna16"`` are re-registered
   (vllm/model_executor/layers/quantization/__init__.py:59-106: a registered config replaces the
   built-in of the same name).  vLLM started without ``--quantization`` turns every AWQ
   checkpoint into ``awq_marlin`` (awq_marlin.py:249-278), so that name has to be covered for the
   kernels to be reached at all.  Both configs hand out
     * ``B200AWQLinearMethod`` for linear layers: vLLM's own ``create_weights`` (the checkpoint
       loaders keep working), no Marlin repack, ``apply`` = one fused kernel family for every
       token count (awq.py:262-286 switches to dequantize + matmul at 256 tokens);
     * ``B200AWQMoEMethod`` for fused-MoE layers: the AWQ-layout stacked parameters of
       awq_marlin.py:549-623 kept as they are, ``apply`` with the signature of
       fused_moe_method_base.py:163-172 calling the expert kernels of this package.
   Under ``--quantization moe_wna16`` the expert layers keep that method's parameter layout
   and loader (uint8 [E, N, K/2], moe_wna16.py:252-324,387-512) and are converted back to the
   AWQ layout once after loading (``B200MoeWNA16Method``).
   Layers the kernels cannot take (group sizes other than 32/64/128 for experts, odd hidden
   sizes) fall back to what stock vLLM would have picked.
2. **Operator overrides.**  ``torch.ops._C.awq_gemm`` / ``awq_dequantize`` are re-implemented for
   the CUDA dispatch key with ``allow_override=True`` so that any remaining call site that uses
   the literal op names (vllm/_custom_ops.py:542-605) lands here too.

Options (keyword arguments of ``register`` or the environment variables in brackets, which is
what a vLLM that loads the plug-in itself sees):
  repack_decode  [AWQ_B200_REPACK_DECODE=1]  decode-layout copies of ``qweight`` for <= 8 tokens
  decode_kmajor  [AWQ_B200_DECODE_KMAJOR=1]  K-major copies of the largest layers for 9..16 tokens
  dummy_fill     [AWQ_B200_DUMMY_FILL=seed]  after loading, overwrite the integer parameters and
                 scales from a seeded generator: ``--load-format dummy`` leaves integer
                 parameters uninitialised (model_loader/weight_utils.py:1484-1490) and draws
                 float ones from +-1e-3, not the nibble-uniform / scale-uniform[0.002, 0.02]
                 distributions of the benchmark.
  mode           [AWQ_B200_MODE=kernels|fill_only]  fill_only leaves vLLM's own methods in place
                 and only applies the seeded fill before them (the stock column of a comparison)
``calls`` counts how often each method ran (for tests that must see these kernels, not vLLM's).
"""
from __future__ import annotations

import os
import zlib

import torch

from . import ops

_registered = False
_lib_handle = None
_options = {"repack_decode": False, "decode_kmajor": False, "dummy_fill": None}
calls = {"linear": 0, "moe": 0, "awq_gemm_op": 0, "awq_dequantize_op": 0}


def _awq_gemm(input, qweight, scales, qzeros, split_k_iters):
    calls["awq_gemm_op"] += 1
    return ops.awq_gemm(input.contiguous(), qweight, scales, qzeros, int(split_k_iters))


def _awq_dequantize(qweight, scales, zeros, split_k_iters, thx, thy):
    calls["awq_dequantize_op"] += 1
    return ops.awq_dequantize(qweight, scales, zeros, int(split_k_iters), int(thx), int(thy))


def fill_awq_tensors(qweight, scales, qzeros, seed: int) -> None:
    """Seeded benchmark distributions, in place: nibbles uniform 0..15, scales uniform
    [0.002, 0.02].  Drawn on the parameters' device."""
    gen = torch.Generator(device=qweight.device).manual_seed(int(seed))
    for t in (qweight, qzeros):
        t.copy_(torch.randint(-(2 ** 31), 2 ** 31, t.shape, dtype=torch.int64, device=t.device,
                              generator=gen).to(torch.int32))
    scales.copy_((0.002 + 0.018 * torch.rand(scales.shape, device=scales.device, generator=gen))
                 .to(scales.dtype))


def _name_seed(layer) -> int:
    """A per-layer offset that is the same in every process (str hashes are salted)."""
    return zlib.crc32(str(getattr(layer, "prefix", getattr(layer, "layer_name", ""))).encode())


def _build_methods():
    """Import the vLLM-derived classes (heavy: vLLM's layer modules) and register the configs."""
    from vllm.model_executor.layers.quantization import register_quantization_config

    from . import vllm_methods as vm
    register_quantization_config("awq")(vm.B200AWQConfig)
    register_quantization_config("awq_marlin")(vm.B200AWQMarlinConfig)
    register_quantization_config("moe_wna16")(vm.B200MoeWNA16Config)
    return {"linear": vm.B200AWQLinearMethod, "moe": vm.B200AWQMoEMethod,
            "awq": vm.B200AWQConfig, "awq_marlin": vm.B200AWQMarlinConfig,
            "moe_wna16": vm.B200MoeWNA16Config, "moe_wna16_method": vm.B200MoeWNA16Method}


classes: dict = {}


def _install_fill_only() -> None:
    """Stock vLLM methods, same weights: the seeded fill runs before vLLM's own
    ``process_weights_after_loading`` (Marlin repack included), nothing else changes.  This is
    the stock column of the serving comparison."""
    from vllm.model_executor.layers.quantization.awq import AWQLinearMethod
    from vllm.model_executor.layers.quantization.awq_marlin import (AWQMarlinLinearMethod,
                                                                    AWQMarlinMoEMethod)

    def wrap_linear(cls):
        stock = cls.process_weights_after_loading

        def process(self, layer):
            if _options["dummy_fill"] is not None:
                fill_awq_tensors(layer.qweight.data, layer.scales.data, layer.qzeros.data,
                                 _options["dummy_fill"] + _name_seed(layer))
            return stock(self, layer)

        cls.process_weights_after_loading = process

    wrap_linear(AWQLinearMethod)
    wrap_linear(AWQMarlinLinearMethod)
    stock_moe = AWQMarlinMoEMethod.process_weights_after_loading

    def process_moe(self, layer):
        if _options["dummy_fill"] is not None:
            seed = _options["dummy_fill"] + _name_seed(layer)
            fill_awq_tensors(layer.w13_qweight.data, layer.w13_scales.data,
                             layer.w13_qzeros.data, seed + 1)
            fill_awq_tensors(layer.w2_qweight.data, layer.w2_scales.data,
                             layer.w2_qzeros.data, seed + 2)
        return stock_moe(self, layer)

    AWQMarlinMoEMethod.process_weights_after_loading = process_moe


def register(full_gemm: bool = True, repack_decode: bool = False, decode_kmajor: bool = False,
             dummy_fill: int | None = None, mode: str | None = None) -> None:
    """Install the hooks.  Needs vLLM's compiled ops to be importable (the op schemas are defined
    by vllm._C).  ``mode`` [AWQ_B200_MODE]: "kernels" (default: both hooks of the module text) or
    "fill_only" (stock vLLM kernels on the seeded weights).  ``full_gemm`` is kept for callers of
    the earlier signature: the linear method uses the fused kernels for every token count."""
    global _registered, _lib_handle
    env = os.environ.get
    _options["repack_decode"] = repack_decode or env("AWQ_B200_REPACK_DECODE") == "1"
    _options["decode_kmajor"] = decode_kmajor or env("AWQ_B200_DECODE_KMAJOR") == "1"
    if dummy_fill is None and env("AWQ_B200_DUMMY_FILL") not in (None, ""):
        dummy_fill = int(env("AWQ_B200_DUMMY_FILL"))
    _options["dummy_fill"] = dummy_fill
    if _registered:
        return
    mode = mode or env("AWQ_B200_MODE") or "kernels"
    if mode == "fill_only":
        _install_fill_only()
        _registered = True
        return
    if mode != "kernels":
        raise ValueError("mode is 'kernels' or 'fill_only'")
    import vllm._C  # noqa: F401  (defines the _C op schemas)
    lib = torch.library.Library("_C", "IMPL")
    lib.impl("awq_gemm", _awq_gemm, "CUDA", allow_override=True)
    lib.impl("awq_dequantize", _awq_dequantize, "CUDA", allow_override=True)
    _lib_handle = lib  # keep the registration alive
    classes.update(_build_methods())
    _registered = True
