"""The plug-in under vLLM's own layer classes, the way a server started with no --quantization
flag reaches them: the checkpoint's ``quantization_config`` says "awq", vLLM's override probe
turns that into "awq_marlin" (config/model.py:1046-1068), ``get_quantization_config`` hands back
the class the plug-in registered, and vLLM's ``QKVParallelLinear`` / ``RowParallelLinear`` /
``FusedMoE`` ask it for their quant methods.  The layers then run this package's kernels (call
counters + device status) and agree with the CPU oracle."""
import socket

import numpy as np
import pytest
import torch

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2
HF_QUANT = {"quant_method": "awq", "bits": 4, "group_size": 128, "zero_point": True,
            "version": "gemm"}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def env(built_library):
    """A one-rank vLLM process state: current VllmConfig, distributed groups of size 1."""
    try:
        import vllm._C  # noqa: F401
        import vllm._moe_C  # noqa: F401
        from vllm.config import VllmConfig, set_current_vllm_config
        from vllm.distributed import (destroy_distributed_environment, destroy_model_parallel,
                                      init_distributed_environment, initialize_model_parallel)
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm not usable here: {e}")
    from awq_b200 import vllm_plugin
    vllm_plugin.register()
    cfg = VllmConfig()
    ctx = set_current_vllm_config(cfg)
    ctx.__enter__()
    torch.cuda.set_device(0)
    init_distributed_environment(world_size=1, rank=0, local_rank=0, backend="nccl",
                                 distributed_init_method=f"tcp://127.0.0.1:{_free_port()}")
    initialize_model_parallel(1, 1)
    try:
        yield cfg
    finally:
        destroy_model_parallel()
        destroy_distributed_environment()
        ctx.__exit__(None, None, None)


def _resolve_quant_config(user_quant=None):
    """vLLM's probe for a checkpoint whose config says "awq" (config/model.py:1046-1068)."""
    from vllm.model_executor.layers.quantization import get_quantization_config
    name = get_quantization_config("awq_marlin").override_quantization_method(HF_QUANT,
                                                                               user_quant)
    if name is None and user_quant is not None:
        name = get_quantization_config(user_quant).override_quantization_method(
            HF_QUANT, user_quant) or user_quant
    if name is None:
        name = HF_QUANT["quant_method"]
    return name, get_quantization_config(name).from_config(HF_QUANT)


def _status() -> int:
    import ctypes
    from awq_b200 import _lib
    v = ctypes.c_int(-1)
    _lib.check("awq_b200_device_status", _lib.load().awq_b200_device_status(ctypes.byref(v)))
    return v.value


@pytest.mark.parametrize("user_quant", [None, "awq"])
def test_registered_configs_are_what_vllm_resolves(env, user_quant):
    from awq_b200 import vllm_plugin
    name, qc = _resolve_quant_config(user_quant)
    assert name == ("awq_marlin" if user_quant is None else "awq")
    assert type(qc) is vllm_plugin.classes[name]


def test_vllm_linear_layers_run_our_kernels(env):
    from vllm.model_executor.layers.linear import QKVParallelLinear, RowParallelLinear
    from awq_b200 import synth, vllm_plugin
    _, qc = _resolve_quant_config()
    hidden, heads, kv_heads, head_dim = 2048, 16, 4, 128
    qkv = QKVParallelLinear(hidden, head_dim, heads, kv_heads, bias=True, quant_config=qc,
                            params_dtype=torch.float16, prefix="model.layers.0.self_attn.qkv_proj")
    o = RowParallelLinear(heads * head_dim, hidden, bias=False, quant_config=qc,
                          params_dtype=torch.float16, prefix="model.layers.0.self_attn.o_proj")
    assert type(qkv.quant_method) is vllm_plugin.classes["linear"]
    assert type(o.quant_method) is vllm_plugin.classes["linear"]
    for layer, (k, n), seed in ((qkv, (hidden, (heads + 2 * kv_heads) * head_dim), 3),
                                (o, (heads * head_dim, hidden), 4)):
        qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=seed)
        assert tuple(layer.qweight.shape) == tuple(qw.shape)
        assert tuple(layer.scales.shape) == tuple(s.shape)
        layer.cuda()
        layer.qweight.data.copy_(qw)
        layer.scales.data.copy_(s)
        layer.qzeros.data.copy_(qz)
        bias = None
        if layer.bias is not None:
            bias = torch.randn(n, generator=torch.Generator().manual_seed(seed)).half()
            layer.bias.data.copy_(bias)
        layer.quant_method.process_weights_after_loading(layer)
        w = O.dequantize_fp32(qw.numpy(), s.numpy(), qz.numpy(), 128)
        for m in (1, 16, 300):
            x = synth.activations(m, k, seed=m)
            before = vllm_plugin.calls["linear"]
            with torch.inference_mode():
                y = layer(x.cuda())
            y = y[0] if isinstance(y, tuple) else y
            assert vllm_plugin.calls["linear"] == before + 1
            assert y.shape == (m, n) and y.dtype == torch.float16
            ref = x.numpy().astype(np.float32) @ w
            if bias is not None:
                ref = ref + bias.numpy().astype(np.float32)
            assert O.rel_err(y.float().cpu().numpy(), ref) < TOL
    assert _status() == 0


def test_linear_op_traces_under_torch_compile(env):
    """vLLM compiles the model with fullgraph=True: the method's apply must trace as one
    registered operator, with a symbolic token count."""
    from vllm.model_executor.layers.quantization.awq import AWQConfig
    from awq_b200 import synth, vllm_plugin
    k, n = 1024, 768
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=9)
    method = vllm_plugin.classes["linear"](AWQConfig(4, 128, True))

    class Layer(torch.nn.Module):
        def forward(self, x):
            return method.apply(self, x)

    layer = Layer()
    layer.qweight = torch.nn.Parameter(qw.cuda(), requires_grad=False)
    layer.scales = torch.nn.Parameter(s.cuda(), requires_grad=False)
    layer.qzeros = torch.nn.Parameter(qz.cuda(), requires_grad=False)
    method.process_weights_after_loading(layer)
    compiled = torch.compile(layer, fullgraph=True, dynamic=True, backend="eager")
    w = O.dequantize_fp32(qw.numpy(), s.numpy(), qz.numpy(), 128)
    for m in (3, 40):
        x = synth.activations(m, k, seed=m)
        y = compiled(x.cuda())
        assert O.rel_err(y.float().cpu().numpy(), x.numpy().astype(np.float32) @ w) < TOL


@pytest.mark.parametrize("t", [1, 16, 200])
def test_vllm_fused_moe_layer_runs_our_kernels(env, t):
    from vllm.forward_context import set_forward_context
    from vllm.model_executor.layers.fused_moe import FusedMoE
    from awq_b200 import synth, vllm_plugin
    _, qc = _resolve_quant_config()
    e, topk, h, inter = 32, 4, 1024, 384
    moe = FusedMoE(num_experts=e, top_k=topk, hidden_size=h, intermediate_size=inter,
                   params_dtype=torch.float16, renormalize=True, quant_config=qc,
                   prefix=f"model.layers.{t}.mlp.experts")
    assert type(moe.quant_method) is vllm_plugin.classes["moe"]
    w1, w2 = synth.moe_layer_tensors(e, h, inter, 128, seed=11)
    assert tuple(moe.w13_qweight.shape) == tuple(w1[0].shape)
    assert tuple(moe.w2_qweight.shape) == tuple(w2[0].shape)
    assert tuple(moe.w13_scales.shape) == tuple(w1[1].shape)
    assert tuple(moe.w2_qzeros.shape) == tuple(w2[2].shape)
    moe.cuda()
    for name, src in (("w13_qweight", w1[0]), ("w13_scales", w1[1]), ("w13_qzeros", w1[2]),
                      ("w2_qweight", w2[0]), ("w2_scales", w2[1]), ("w2_qzeros", w2[2])):
        getattr(moe, name).data.copy_(src)
    moe.quant_method.process_weights_after_loading(moe)
    x = synth.activations(t, h, seed=t)
    logits = torch.randn(t, e, generator=torch.Generator().manual_seed(t))
    before = vllm_plugin.calls["moe"]
    with torch.inference_mode(), set_forward_context(None, env, num_tokens=t):
        y = moe(x.cuda(), logits.cuda())
    assert vllm_plugin.calls["moe"] == before + 1
    assert y.shape == (t, h) and y.dtype == torch.float16
    wts, ids, _ = O.topk_softmax(logits.numpy(), topk, True)
    ref = O.fused_experts_fp32(x.numpy(), *[a.numpy() for a in w1], *[a.numpy() for a in w2],
                               wts, ids, 128)
    assert O.rel_err(y.float().cpu().numpy(), ref) < TOL
    assert _status() == 0


def test_moe_wna16_route_runs_our_kernels(env):
    """--quantization moe_wna16 on an AWQ checkpoint: vLLM's MoeWNA16 parameters and loader, the
    plug-in's method; the layer is loaded with tensors in that method's byte layout."""
    from vllm.forward_context import set_forward_context
    from vllm.model_executor.layers.fused_moe import FusedMoE
    from awq_b200 import synth, vllm_plugin
    name, qc = _resolve_quant_config("moe_wna16")
    assert name == "moe_wna16" and type(qc) is vllm_plugin.classes["moe_wna16"]
    e, topk, h, inter, t = 16, 4, 512, 256, 24
    moe = FusedMoE(num_experts=e, top_k=topk, hidden_size=h, intermediate_size=inter,
                   params_dtype=torch.float16, renormalize=True, quant_config=qc,
                   prefix="model.layers.77.mlp.experts")
    assert type(moe.quant_method) is vllm_plugin.classes["moe_wna16_method"]
    assert moe.w13_qweight.dtype == torch.uint8
    assert tuple(moe.w13_qweight.shape) == (e, 2 * inter, h // 2)
    w1, w2 = synth.moe_layer_tensors(e, h, inter, 128, seed=21)
    moe.cuda()
    for proj, (qw, sc, qz) in (("w13", w1), ("w2", w2)):
        getattr(moe, proj + "_qweight").data.copy_(torch.from_numpy(
            np.stack([O.awq_to_wna16_qweight(a) for a in qw.numpy()])))
        getattr(moe, proj + "_qzeros").data.copy_(torch.from_numpy(
            np.stack([O.awq_to_wna16_qzeros(a) for a in qz.numpy()])))
        getattr(moe, proj + "_scales").data.copy_(sc.transpose(1, 2))
    moe.quant_method.process_weights_after_loading(moe)
    assert moe.w13_qweight.dtype == torch.int32 and torch.equal(moe.w13_qweight.cpu(), w1[0])
    assert torch.equal(moe.w2_qzeros.cpu(), w2[2])
    x = synth.activations(t, h, seed=t)
    logits = torch.randn(t, e, generator=torch.Generator().manual_seed(t))
    before = vllm_plugin.calls["moe"]
    with torch.inference_mode(), set_forward_context(None, env, num_tokens=t):
        y = moe(x.cuda(), logits.cuda())
    assert vllm_plugin.calls["moe"] == before + 1
    wts, ids, _ = O.topk_softmax(logits.numpy(), topk, True)
    ref = O.fused_experts_fp32(x.numpy(), *[a.numpy() for a in w1], *[a.numpy() for a in w2],
                               wts, ids, 128)
    assert O.rel_err(y.float().cpu().numpy(), ref) < TOL
    assert _status() == 0


def test_dummy_fill_gives_benchmark_distributions(env):
    """--load-format dummy leaves integer parameters uninitialised; with dummy_fill the method
    draws nibble-uniform words and scales uniform in [0.002, 0.02], the same in every process."""
    from vllm.model_executor.layers.linear import RowParallelLinear
    from awq_b200 import vllm_plugin
    _, qc = _resolve_quant_config()
    vllm_plugin.register(dummy_fill=7)
    try:
        layers = [RowParallelLinear(1024, 512, bias=False, quant_config=qc,
                                    params_dtype=torch.float16,
                                    prefix="model.layers.3.mlp.down_proj").cuda() for _ in range(2)]
        for layer in layers:
            layer.quant_method.process_weights_after_loading(layer)
        assert torch.equal(layers[0].qweight, layers[1].qweight)
        q = torch.from_numpy(O.unpack_awq(layers[0].qweight.cpu().numpy()).astype(np.int64))
        counts = torch.bincount(q.flatten(), minlength=16).float()
        assert counts.min() > 0.9 * counts.mean() and counts.max() < 1.1 * counts.mean()
        s = layers[0].scales.float()
        assert 0.002 <= s.min().item() and s.max().item() <= 0.0201
        with torch.inference_mode():
            y = layers[0](torch.ones(4, 1024, dtype=torch.float16, device="cuda"))
        y = y[0] if isinstance(y, tuple) else y
        assert torch.isfinite(y).all()
    finally:
        vllm_plugin.register()
