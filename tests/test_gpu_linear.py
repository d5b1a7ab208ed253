"""Parity of the CUDA AWQ linear kernels (through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu

TOL = 1e-2  # max |y - ref| / max |ref|, fp16 output with fp32 accumulation


@pytest.fixture(scope="module")
def A(built_library):
    import awq_b200
    assert torch.cuda.is_available()
    return awq_b200


def dev(*ts):
    return [torch.from_numpy(np.ascontiguousarray(t)).cuda() if isinstance(t, np.ndarray)
            else t.cuda() for t in ts]


def check_gemm(A, x, qw, s, qz, group, kernel, bias=None):
    ref = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy(), group)
    if bias is not None:
        ref = ref + bias.numpy().astype(np.float32)
    xd, qwd, sd, qzd = dev(x, qw, s, qz)
    bd = bias.cuda() if bias is not None else None
    y = A.awq_gemm(xd, qwd, sd, qzd, 8, bias=bd, kernel=kernel)
    torch.cuda.synchronize()
    y = y.cpu().numpy()
    assert y.shape == ref.shape and y.dtype == np.float16
    assert np.isfinite(y.astype(np.float32)).all()
    err = O.rel_err(y, ref)
    assert err < TOL, f"rel err {err}"
    assert O.elementwise_ok(y, ref, TOL)
    return err


CASES = ["tiny", "ragged_m", "two_groups", "wide", "g64"]


@pytest.mark.parametrize("name", CASES)
def test_dequantize_golden_bit_exact(A, golden, name):
    qw, s, qz = dev(golden[f"{name}.qweight"], golden[f"{name}.scales"], golden[f"{name}.qzeros"])
    w = A.awq_dequantize(qw, s, qz, 0, 0, 0).cpu().numpy()
    assert np.array_equal(w.view(np.uint16), golden[f"{name}.w_fp16"].view(np.uint16))


@pytest.mark.parametrize("k,n,g", [(8192, 8192, 128), (1024, 10240, 128), (384, 72, 64),
                                   (29568, 1024, 128)])
def test_dequantize_bit_exact_vs_oracle(A, k, n, g):
    from awq_b200 import synth
    qw, s, qz = synth.awq_linear_tensors(k, n, g, seed=3)
    w = A.awq_dequantize(*dev(qw, s, qz), 0, 0, 0).cpu().numpy()
    ref = O.dequantize_fp16(qw.numpy(), s.numpy(), qz.numpy(), g)
    assert np.array_equal(w.view(np.uint16), ref.view(np.uint16))


def test_unpack_index_known_answer(A):
    """Word 0x75316420 with zero point 0 and scale 1 dequantises to columns 0..7."""
    qw = torch.tensor([[0x75316420]], dtype=torch.int32).repeat(8, 1)
    qz = torch.zeros(1, 1, dtype=torch.int32)
    s = torch.ones(1, 8, dtype=torch.float16)
    w = A.awq_dequantize(*dev(qw, s, qz), 0, 0, 0).cpu()
    assert w[0].tolist() == [float(i) for i in range(8)]


@pytest.mark.parametrize("name", CASES)
def test_gemm_golden_generic(A, golden, name):
    import awq_b200
    g = int(golden[f"{name}.group"][0])
    x, qw, s, qz = (torch.from_numpy(golden[f"{name}.{k}"]) for k in
                    ("x", "qweight", "scales", "qzeros"))
    check_gemm(A, x, qw, s, qz, g, awq_b200.KERNEL_GENERIC)
    check_gemm(A, x, qw, s, qz, g, awq_b200.KERNEL_AUTO)


def _kernels(A):
    return {"stream": A.KERNEL_STREAM, "stream_exact": A.KERNEL_STREAM_EXACT}


@pytest.mark.parametrize("kern", ["stream", "stream_exact"])
@pytest.mark.parametrize("m,k,n,g", [
    (1, 128, 32, 128), (1, 256, 256, 128), (3, 512, 64, 128), (8, 1024, 288, 128),
    (9, 1024, 512, 128), (16, 8192, 1024, 128), (16, 2048, 1536, 128), (17, 768, 2048, 128),
    (32, 1152, 320, 128), (5, 256, 96, 64), (16, 384, 256, 32), (4, 3712, 8192, 128),
])
def test_gemm_stream_vs_oracle(A, kern, m, k, n, g):
    from awq_b200 import synth
    qw, s, qz = synth.awq_linear_tensors(k, n, g, seed=m + k)
    x = synth.activations(m, k, seed=n)
    check_gemm(A, x, qw, s, qz, g, _kernels(A)[kern])


def test_gemm_stream_bias_and_determinism(A):
    from awq_b200 import synth
    m, k, n = 16, 2048, 768
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=11)
    x = synth.activations(m, k, seed=12)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(5)).half()
    check_gemm(A, x, qw, s, qz, 128, A.KERNEL_STREAM, bias=bias)
    xd, qwd, sd, qzd = dev(x, qw, s, qz)
    y1 = A.awq_gemm(xd, qwd, sd, qzd, 8)
    y2 = A.awq_gemm(xd, qwd, sd, qzd, 8)
    assert torch.equal(y1, y2)


def test_gemm_stream_outliers_and_extreme_nibbles(A):
    """All-15 weights with all-0 zeros, all-0 weights with all-15 zeros, large activations."""
    m, k, n = 8, 512, 256
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(1)).half()
    x[:, ::37] *= 60.0
    s = torch.full((k // 128, n), 0.02, dtype=torch.float16)
    full = torch.full((k, n // 8), -1, dtype=torch.int32)        # every nibble 15
    zero = torch.zeros((k, n // 8), dtype=torch.int32)
    for qw, qz in [(full, zero[:k // 128]), (zero, full[:k // 128])]:
        for kern in (A.KERNEL_STREAM, A.KERNEL_STREAM_EXACT):
            check_gemm(A, x, qw.contiguous(), s, qz.contiguous(), 128, kern)


def test_linear_method_apply_shapes(A):
    from awq_b200 import AWQConfig, AWQLinear, AWQLinearMethod, synth
    k, n = 1024, 512
    method = AWQLinearMethod(AWQConfig(group_size=128))
    layer = AWQLinear()
    method.create_weights(layer, k, [n], k, n, torch.float16, device="cuda")
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=21)
    layer.qweight.data.copy_(qw); layer.scales.data.copy_(s); layer.qzeros.data.copy_(qz)
    method.process_weights_after_loading(layer)
    x = synth.activations(6, k, seed=22).reshape(2, 3, k)
    y = method.apply(layer, x.cuda())
    assert y.shape == (2, 3, n)
    ref = O.awq_linear(x.reshape(6, k).numpy(), qw.numpy(), s.numpy(), qz.numpy())
    assert O.rel_err(y.reshape(6, n).cpu().numpy(), ref) < TOL
    assert method.apply(layer, torch.empty(0, k, dtype=torch.float16, device="cuda")).shape == (0, n)


def test_linearity_property_full_size(A):
    """Size-independent check at a benchmark shape: f(a x1 + x2) rows vs a f(x1) + f(x2)
    computed from two launches, and the M=1 row equals row 0 of the M=16 launch."""
    from awq_b200 import synth
    k, n = 8192, 10240
    qw, s, qz = dev(*synth.awq_linear_tensors(k, n, 128, seed=0))
    x = synth.activations(16, k, seed=0).cuda()
    y16 = A.awq_gemm(x, qw, s, qz, 8).float()
    y1 = A.awq_gemm(x[:1].contiguous(), qw, s, qz, 8).float()
    assert O.rel_err(y1.cpu().numpy(), y16[:1].cpu().numpy()) < 2e-3
    x2 = (x[:8] * 0.5 + x[8:] * 0.25).half()
    y2 = A.awq_gemm(x2, qw, s, qz, 8).float()
    lin = 0.5 * y16[:8] + 0.25 * y16[8:]
    assert O.rel_err(y2.cpu().numpy(), lin.cpu().numpy()) < 5e-3


def test_against_installed_vllm_kernels(A):
    """Live comparison with the kernels the reference harness actually runs, when the vLLM
    wheel's compiled ops load on this box."""
    try:
        from vllm import _custom_ops as vops
        import vllm._C  # noqa: F401
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm compiled ops unavailable: {e}")
    from awq_b200 import synth
    k, n = 1024, 512
    qw, s, qz = dev(*synth.awq_linear_tensors(k, n, 128, seed=31))
    w_ref = vops.awq_dequantize(qw, s, qz, 0, 0, 0)
    w = A.awq_dequantize(qw, s, qz, 0, 0, 0)
    assert torch.equal(w, w_ref)
    x = synth.activations(8, k, seed=32).cuda()
    y_ref = vops.awq_gemm(x, qw, s, qz, 8)
    y = A.awq_gemm(x, qw, s, qz, 8)
    assert O.rel_err(y.cpu().numpy(), y_ref.float().cpu().numpy()) < TOL


@pytest.mark.parametrize("m", [1, 8, 16, 64])
def test_back_to_back_layers_see_each_others_outputs(A, m):
    """The decode kernels start before the kernel ahead of them in the stream has finished
    (programmatic dependent launch) and prefetch weights meanwhile.  A chain in which every
    layer reads the output of the one before, launched without any host synchronisation, must
    give exactly what the same chain gives with a device synchronisation after every layer."""
    from awq_b200 import synth
    dims = [(2048, 2048), (2048, 4096), (4096, 2048), (2048, 2048)]
    layers = [[t.cuda() for t in synth.awq_linear_tensors(k, n, 128, seed=40 + i)]
              for i, (k, n) in enumerate(dims)]
    x0 = (synth.activations(m, dims[0][0], seed=m) * 0.25).cuda()

    def chain(sync):
        y = x0
        for qw, s, qz in layers:
            y = A.awq_gemm(y, qw, s, qz, 8)
            y = y * 0.03125  # an elementwise kernel between the layers, as a model has
            if sync:
                torch.cuda.synchronize()
        return y

    want = chain(True)
    assert torch.isfinite(want.float()).all() and want.float().abs().max() > 0
    for _ in range(10):
        got = chain(False)
        assert torch.equal(got, want)
    # and straight from one linear into the next, no kernel in between
    for _ in range(10):
        y = x0
        outs = []
        for qw, s, qz in layers[:1] + layers[3:]:
            y = A.awq_gemm(y, qw, s, qz, 8)
            outs.append(y)
        torch.cuda.synchronize()
        ref = x0
        for (qw, s, qz), o in zip(layers[:1] + layers[3:], outs):
            ref = A.awq_gemm(ref, qw, s, qz, 8)
            torch.cuda.synchronize()
            assert torch.equal(ref, o)
