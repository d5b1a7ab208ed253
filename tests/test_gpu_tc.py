"""Parity of the tcgen05 / TMEM large-M kernel (through the C ABI) with the CPU oracle."""
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
    rc = _lib.load().awq_b200_device_status(ctypes.byref(v))
    assert rc == 0
    return v.value


def run_case(A, m, k, n, g, seed=0, bias=False):
    from awq_b200 import synth
    qw, s, qz = synth.awq_linear_tensors(k, n, g, seed=seed)
    x = synth.activations(m, k, seed=seed + 1)
    b = torch.randn(n, generator=torch.Generator().manual_seed(seed)).half() if bias else None
    y = A.awq_gemm(x.cuda(), qw.cuda(), s.cuda(), qz.cuda(), 8,
                   bias=b.cuda() if bias else None, kernel=A.KERNEL_TCGEN05)
    torch.cuda.synchronize()
    assert device_status() == 0, "a bounded wait in the tcgen05 kernel ran out"
    ref = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy(), g)
    if bias:
        ref = ref + b.numpy().astype(np.float32)
    y = y.cpu().numpy()
    assert np.isfinite(y.astype(np.float32)).all()
    err = O.rel_err(y, ref)
    assert err < TOL, f"rel err {err}"
    assert O.elementwise_ok(y, ref, TOL)


def test_tc_single_stage(A):
    run_case(A, 128, 64, 256, 64)


def test_tc_two_stages_one_group(A):
    run_case(A, 128, 128, 256, 128)


@pytest.mark.parametrize("m,k,n,g", [
    (128, 512, 128, 128),      # 128-column tile
    (1, 256, 32, 128),         # single token, N tail inside a tile
    (300, 1024, 512, 128),     # ragged M
    (64, 2048, 1536, 128),
    (257, 512, 288, 128),      # N not a multiple of the tile
    (1024, 8192, 1024, 128),   # long K: many ring rounds
    (256, 256, 2048, 64),      # group 64
    (4096, 1024, 2048, 128),   # many tiles, 256-column path
])
def test_tc_vs_oracle(A, m, k, n, g):
    run_case(A, m, k, n, g, seed=m + n)


def test_tc_bias_and_auto_dispatch(A):
    from awq_b200 import synth
    run_case(A, 200, 512, 256, 128, seed=5, bias=True)
    # AUTO picks the tcgen05 kernel above the streaming kernel's range
    k, n, m = 1024, 512, 96
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=9)
    x = synth.activations(m, k, seed=10)
    y = A.awq_gemm(x.cuda(), qw.cuda(), s.cuda(), qz.cuda(), 8).cpu().numpy()
    ref = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy(), 128)
    assert O.rel_err(y, ref) < TOL
    assert device_status() == 0


def test_tc_matches_dequantize_then_matmul(A):
    """Same operands through awq_dequantize + torch.matmul (the reference's >= 256-token path,
    quantization/awq.py:276-281): the fused kernel multiplies the same fp16 weights."""
    from awq_b200 import synth
    m, k, n = 512, 2048, 1024
    qw, s, qz = [a.cuda() for a in synth.awq_linear_tensors(k, n, 128, seed=3)]
    x = synth.activations(m, k, seed=4).cuda()
    w = A.awq_dequantize(qw, s, qz, 0, 0, 0)
    ref = (x.float() @ w.float()).cpu().numpy()
    y = A.awq_gemm(x, qw, s, qz, 8, kernel=A.KERNEL_TCGEN05).cpu().numpy()
    assert O.rel_err(y, ref) < 2e-3
