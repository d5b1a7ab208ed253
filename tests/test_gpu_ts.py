"""Parity of the decode-size tcgen05 kernel (weights registers -> TMEM, A operand in TMEM) with
the CPU oracle, through the C ABI."""
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


def run_case(A, kernel, m, k, n, seed=0, bias=False):
    from awq_b200 import synth
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=seed)
    x = synth.activations(m, k, seed=seed + 1)
    b = torch.randn(n, generator=torch.Generator().manual_seed(seed)).half() if bias else None
    y = A.awq_gemm(x.cuda(), qw.cuda(), s.cuda(), qz.cuda(), 8,
                   bias=b.cuda() if bias else None, kernel=kernel)
    torch.cuda.synchronize()
    assert device_status() == 0, "a bounded wait ran out"
    ref = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy(), 128)
    if bias:
        ref = ref + b.numpy().astype(np.float32)
    y = y.cpu().numpy()
    assert np.isfinite(y.astype(np.float32)).all()
    err = O.rel_err(y, ref)
    assert err < TOL, f"rel err {err}"
    assert O.elementwise_ok(y, ref, TOL)


SHAPES = [
    (16, 128, 256),     # one stage, one slab
    (16, 256, 256),     # two stages
    (16, 1024, 512),    # ring wraps, two slabs
    (1, 512, 256), (3, 384, 32), (9, 640, 288),   # ragged M, N edge inside a slab
    (16, 8192, 8192), (4, 3712, 8192), (16, 2048, 1536),
]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_ts_exact_vs_oracle(A, m, k, n):
    run_case(A, A.KERNEL_TS_EXACT, m, k, n, seed=m + n)


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_ts_fast_vs_oracle(A, m, k, n):
    run_case(A, A.KERNEL_TS, m, k, n, seed=m + k)


def test_ts_bias_determinism_and_agreement_with_stream_kernel(A):
    from awq_b200 import synth
    run_case(A, A.KERNEL_TS, 16, 2048, 768, seed=4, bias=True)
    m, k, n = 16, 4096, 2048
    qw, s, qz = [a.cuda() for a in synth.awq_linear_tensors(k, n, 128, seed=8)]
    x = synth.activations(m, k, seed=9).cuda()
    y1 = A.awq_gemm(x, qw, s, qz, 8, kernel=A.KERNEL_TS)
    y2 = A.awq_gemm(x, qw, s, qz, 8, kernel=A.KERNEL_TS)
    assert torch.equal(y1, y2)
    y3 = A.awq_gemm(x, qw, s, qz, 8, kernel=A.KERNEL_STREAM)
    assert O.rel_err(y1.cpu().numpy(), y3.float().cpu().numpy()) < 2e-3
    assert device_status() == 0
