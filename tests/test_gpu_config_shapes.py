"""Oracle parity at the exact shapes the benchmark configurations name, through the kernel the
dispatcher picks (AWQ_B200_KERNEL_AUTO) and through the K-major decode kernel: the single layer
of configuration 1 (M 16, K 8192, N 8192, seed 0) and the four Qwen2.5-72B layers of
configuration 2 at M in {1, 4, 16, 64, 256, 1024} (4096 on o_proj).  The fp32 weight matrix of a
layer is built once and reused for every M."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2

LAYERS = {"qkv": (8192, 10240), "o_proj": (8192, 8192), "gate_up": (8192, 59136),
          "down": (29568, 8192)}
SWEEP_M = (1, 4, 16, 64, 256, 1024)


@pytest.fixture(scope="module")
def A(built_library):
    import awq_b200
    assert torch.cuda.is_available()
    return awq_b200


def device_status():
    from awq_b200 import _lib
    v = ctypes.c_int(-1)
    assert _lib.load().awq_b200_device_status_clear(ctypes.byref(v)) == 0
    return v.value


def check(y, ref):
    y = y.float().cpu().numpy()
    assert np.isfinite(y).all()
    err = O.rel_err(y, ref)
    assert err < TOL, f"rel err {err}"
    assert O.elementwise_ok(y, ref, TOL)


@pytest.fixture(scope="module", params=list(LAYERS))
def layer(request, A):
    """Packed tensors on the GPU and the fp32 dequantised matrix on the host, once per layer."""
    from awq_b200 import synth
    k, n = LAYERS[request.param]
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=0)
    w = torch.from_numpy(O.dequantize_fp32(qw.numpy(), s.numpy(), qz.numpy(), 128))
    dev = (qw.cuda(), s.cuda(), qz.cuda())
    yield request.param, k, n, dev, w
    del w, dev
    torch.cuda.empty_cache()


def test_config2_layer_sweep(A, layer):
    from awq_b200 import synth
    name, k, n, (qw, s, qz), w = layer
    ms = SWEEP_M + ((4096,) if name == "o_proj" else ())
    km = A.awq_repack_kmajor(qw)
    for m in ms:
        x = synth.activations(m, k, seed=m)
        ref = (x.float() @ w).numpy()
        check(A.awq_gemm(x.cuda(), qw, s, qz, 8), ref)
        if m <= 16:
            check(A.awq_gemm(x.cuda(), km, s, qz, 8, kernel=A.KERNEL_Q8), ref)
        assert device_status() == 0, f"{name} M={m}: a bounded wait ran out"


def test_config1_exact(A):
    """x fp16 [16, 8192], qweight int32 [8192, 1024], qzeros [64, 1024], scales [64, 8192],
    seed 0, through AWQLinearMethod.apply."""
    from awq_b200 import synth
    m, k, n = 16, 8192, 8192
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=0)
    assert tuple(qw.shape) == (8192, 1024) and tuple(qz.shape) == (64, 1024)
    assert tuple(s.shape) == (64, 8192)
    x = synth.activations(m, k, seed=0)
    ref = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy(), 128)
    method = A.AWQLinearMethod(A.AWQConfig())
    lin = A.AWQLinear()
    method.create_weights(lin, k, [n], k, n, torch.float16)
    lin.qweight.data.copy_(qw)
    lin.scales.data.copy_(s)
    lin.qzeros.data.copy_(qz)
    method.process_weights_after_loading(lin)
    y = method.apply(lin, x.cuda())
    assert tuple(y.shape) == (16, 8192) and y.dtype == torch.float16
    check(y, ref)
    assert device_status() == 0
