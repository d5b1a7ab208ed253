"""Drop-in check inside the reference's own dependency: vLLM's AWQLinearMethod (unmodified) is run
on a layer once with vLLM's compiled ops and once after awq_b200.vllm_plugin.register() has
re-implemented torch.ops._C.awq_gemm / awq_dequantize; both must agree with each other and with
the oracle."""
import numpy as np
import pytest
import torch

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu


def test_vllm_awq_linear_method_runs_on_our_ops(built_library):
    try:
        import vllm._C  # noqa: F401
        from vllm.model_executor.layers.quantization.awq import AWQConfig, AWQLinearMethod
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm not usable here: {e}")
    from awq_b200 import synth, vllm_plugin
    k, n = 2048, 1536
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=41)
    try:
        cfg = AWQConfig(weight_bits=4, group_size=128, zero_point=True)
    except TypeError:
        cfg = AWQConfig(4, 128, True)
    method = AWQLinearMethod(cfg)

    class Layer(torch.nn.Module):
        pass

    layer = Layer()
    layer.qweight = torch.nn.Parameter(qw.cuda(), requires_grad=False)
    layer.scales = torch.nn.Parameter(s.cuda(), requires_grad=False)
    layer.qzeros = torch.nn.Parameter(qz.cuda(), requires_grad=False)

    results = {}
    for m in (8, 300):   # awq_gemm path and dequantize + matmul path of AWQLinearMethod.apply
        x = synth.activations(m, k, seed=m).cuda()
        results[("vllm", m)] = method.apply(layer, x).float().cpu().numpy()
    vllm_plugin.register()
    vllm_plugin.register()   # idempotent
    for m in (8, 300):
        x = synth.activations(m, k, seed=m).cuda()
        ours = method.apply(layer, x)
        assert ours.shape == (m, n) and ours.dtype == torch.float16
        results[("ours", m)] = ours.float().cpu().numpy()
        ref = O.awq_gemm_fp32(x.cpu().numpy(), qw.numpy(), s.numpy(), qz.numpy(), 128)
        assert O.rel_err(results[("ours", m)], ref) < 1e-2
        assert O.rel_err(results[("ours", m)], results[("vllm", m)]) < 1e-2
    # the literal op names now run this package's kernels
    y = torch.ops._C.awq_gemm(synth.activations(4, k).cuda(), layer.qweight, layer.scales,
                              layer.qzeros, 8)
    assert y.shape == (4, n)


def test_plugin_linear_method_with_layout_copies(built_library):
    """register(repack_decode=True, decode_kmajor=True): the plug-in's linear method keeps the
    decode-layout copy (and, for layers large enough, the K-major copy) after loading and serves
    each token count from the layout made for it."""
    try:
        import vllm._C  # noqa: F401
        from vllm.model_executor.layers.quantization import awq as vllm_awq
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm not usable here: {e}")
    from awq_b200 import synth, vllm_plugin
    vllm_plugin.register(repack_decode=True, decode_kmajor=True)
    try:
        method_cls = vllm_plugin.classes["linear"]
        assert issubclass(method_cls, vllm_awq.AWQLinearMethod)
        cfg = vllm_awq.AWQConfig(weight_bits=4, group_size=128, zero_point=True)
        for (k, n, want_kmajor) in ((2048, 1536, False), (8192, 59136, True)):
            qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=43)
            method = method_cls(cfg)

            class Layer(torch.nn.Module):
                pass

            layer = Layer()
            layer.qweight = torch.nn.Parameter(qw.cuda(), requires_grad=False)
            layer.scales = torch.nn.Parameter(s.cuda(), requires_grad=False)
            layer.qzeros = torch.nn.Parameter(qz.cuda(), requires_grad=False)
            method.process_weights_after_loading(layer)
            assert layer.qweight_decode is not None
            assert layer.qweight_decode.shape == layer.qweight.shape
            assert (layer.qweight_kmajor is not None) == want_kmajor
            w = O.dequantize_fp32(qw.numpy(), s.numpy(), qz.numpy(), 128)
            for m in (1, 8, 9, 16, 300):
                x = synth.activations(m, k, seed=m).cuda()
                y = method.apply(layer, x)
                assert y.shape == (m, n) and y.dtype == torch.float16
                ref = x.cpu().numpy().astype(np.float32) @ w
                assert O.rel_err(y.float().cpu().numpy(), ref) < 1e-2
    finally:
        vllm_plugin.register()   # options back to the defaults
