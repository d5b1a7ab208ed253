"""Parity of the weights-in-tensor-memory tcgen05 kernel (dequantised weights registers -> TMEM as
the A operand, activations as the B operand) with the CPU oracle, through the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def A(built_library):
    import awq_b200
    assert torch.cuda.is_available()
    return awq_b200


def device_status():
    from awq_b200 import _lib
    v = ctypes.c_int(-1)
    assert _lib.load().awq_b200_device_status(ctypes.byref(v)) == 0
    return v.value


def run_case(A, m, k, n, seed=0, bias=False):
    from awq_b200 import synth
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=seed)
    x = synth.activations(m, k, seed=seed + 1)
    b = torch.randn(n, generator=torch.Generator().manual_seed(seed)).half() if bias else None
    y = A.awq_gemm(x.cuda(), qw.cuda(), s.cuda(), qz.cuda(), 8,
                   bias=b.cuda() if bias else None, kernel=A.KERNEL_WT)
    torch.cuda.synchronize()
    assert device_status() == 0, "a bounded wait ran out"
    ref = O.awq_gemm_fp32_torch(x, qw, s, qz, 128).numpy()
    if bias:
        ref = ref + b.numpy().astype(np.float32)
    y = y.cpu().numpy()
    assert np.isfinite(y.astype(np.float32)).all()
    err = O.rel_err(y, ref)
    assert err < TOL, f"rel err {err}"
    assert O.elementwise_ok(y, ref, TOL)


SHAPES = [
    (64, 128, 256),      # one stage, one slab, 64-token tile
    (64, 256, 256),      # two stages: both A ring halves
    (48, 1024, 512),     # ring wraps, ragged M
    (128, 640, 288),     # 128-token tile, N edge inside a slab
    (100, 2048, 1536), (33, 384, 32), (1, 512, 256), (17, 3712, 8192),
    (256, 1024, 1024),   # two token tiles
    (300, 2048, 512),    # ragged last token tile
    (1024, 8192, 1024),
]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_wt_vs_oracle(A, m, k, n):
    run_case(A, m, k, n, seed=m + n)


def test_wt_bias_and_repeat(A):
    run_case(A, 64, 1024, 512, seed=5, bias=True)
    run_case(A, 200, 1024, 512, seed=6, bias=True)


def test_wt_deterministic(A):
    from awq_b200 import synth
    qw, s, qz = [a.cuda() for a in synth.awq_linear_tensors(4096, 2048, 128, seed=3)]
    x = synth.activations(96, 4096, seed=4).cuda()
    y0 = A.awq_gemm(x, qw, s, qz, 8, kernel=A.KERNEL_WT)
    for _ in range(3):
        assert torch.equal(y0, A.awq_gemm(x, qw, s, qz, 8, kernel=A.KERNEL_WT))


def test_wt_rejects_unsupported_shapes(A):
    from awq_b200 import synth
    qw, s, qz = [a.cuda() for a in synth.awq_linear_tensors(256, 264, 128, seed=1)]  # N % 32 != 0
    x = synth.activations(64, 256).cuda()
    with pytest.raises(ValueError):
        A.awq_gemm(x, qw, s, qz, 8, kernel=A.KERNEL_WT)
