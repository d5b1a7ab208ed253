"""Parity of the decode kernel that widens the nibbles with tcgen05.cp and multiplies with int8
MMAs (AWQ_B200_KERNEL_Q8, M <= 16) with the CPU oracle, through the C ABI; bit-exactness of the
K-major repack it reads."""
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


def device_status(clear=True):
    from awq_b200 import _lib
    v = ctypes.c_int(-1)
    fn = _lib.load().awq_b200_device_status_clear if clear else _lib.load().awq_b200_device_status
    assert fn(ctypes.byref(v)) == 0
    return v.value


def run_case(A, m, k, n, seed=0, bias=False, check_pack=True):
    from awq_b200 import synth
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=seed)
    x = synth.activations(m, k, seed=seed + 1)
    km = A.awq_repack_kmajor(qw.cuda())
    if check_pack:
        got = km.cpu().numpy().view(np.uint8).reshape(-1)
        assert np.array_equal(got, O.pack_kmajor(qw.numpy())), "repack is not bit-exact"
    b = torch.randn(n, generator=torch.Generator().manual_seed(seed)).half() if bias else None
    y = A.awq_gemm(x.cuda(), km, s.cuda(), qz.cuda(), 8,
                   bias=b.cuda() if bias else None, kernel=A.KERNEL_Q8)
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
    return y


SHAPES = [
    (16, 128, 256),     # one tile
    (16, 256, 256),     # two groups
    (16, 1024, 512),    # ring wraps, two slabs
    (1, 512, 256), (3, 384, 32), (9, 640, 288),   # ragged M, N edge inside a slab
    (8, 2048, 1536), (16, 8192, 1024), (4, 3840, 8192), (12, 1024, 1280),
    (16, 768, 2048),    # the down projection of a Qwen3-30B-A3B expert
]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_q8_vs_oracle(A, m, k, n):
    run_case(A, m, k, n, seed=m + n, bias=(n == 512))


def test_q8_config1_exact_shape(A):
    """BASELINE config 1: M 16, K 8192, N 8192 (qweight [8192, 1024] words), seed 0."""
    run_case(A, 16, 8192, 8192, seed=0, check_pack=False)


def test_q8_outliers_and_tiny_rows(A):
    """The activations are rewritten as 24-bit fixed point per token: a row with a huge outlier,
    a row of tiny values and an all-zero row must all stay within tolerance."""
    from awq_b200 import synth
    m, k, n = 5, 1024, 512
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=3)
    x = synth.activations(m, k, seed=4)
    x[0, 17] = 3000.0          # outlier 3000 x the typical magnitude
    x[1] *= 1e-3               # tiny row
    x[2] = 0                   # zero row
    x[3, :] = 60000.0          # near the top of the fp16 range
    x[3, ::2] = -60000.0
    km = A.awq_repack_kmajor(qw.cuda())
    y = A.awq_gemm(x.cuda(), km, s.cuda(), qz.cuda(), 8, kernel=A.KERNEL_Q8).cpu().numpy()
    assert device_status() == 0
    ref = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy(), 128)
    for r in range(m):
        scale = np.abs(ref[r]).max()
        if scale == 0:
            assert not y[r].any()
            continue
        if scale > 6e4:        # beyond fp16: the oracle's fp16 result is inf as well
            continue
        assert np.abs(y[r].astype(np.float32) - ref[r]).max() / scale < TOL, f"row {r}"


def test_q8_is_deterministic_and_survives_back_to_back_calls(A):
    """Different weights and activations in consecutive calls that share one scratch buffer and
    are not synchronised: every result must equal the one of an isolated call, bit for bit (the
    partial tiles CTAs hand to each other are summed in a fixed order)."""
    from awq_b200 import synth
    k, n = 8192, 8192
    sets = []
    for i in range(3):
        qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=10 + i)
        sets.append((A.awq_repack_kmajor(qw.cuda()), s.cuda(), qz.cuda()))
    xs = [synth.activations(m, k, seed=20 + m).cuda() for m in (16, 7, 1)]
    refs = []
    for (w, s, qz), x in zip(sets, xs):
        refs.append(A.awq_gemm(x, w, s, qz, 8, kernel=A.KERNEL_Q8).clone())
        torch.cuda.synchronize()
    outs = []
    for it in range(8):
        for (w, s, qz), x in zip(sets, xs):
            outs.append(A.awq_gemm(x, w, s, qz, 8, kernel=A.KERNEL_Q8))
    torch.cuda.synchronize()
    assert device_status() == 0
    for j, o in enumerate(outs):
        assert torch.equal(o, refs[j % 3]), f"call {j} differs from the isolated result"


def test_q8_cold_first_calls(A):
    """First call on freshly written weights, all CTAs starting at once on a cold TLB: loads
    complete out of order there, which is what an odd ring of stages once got wrong."""
    from awq_b200 import synth
    k, n, m = 8192, 8192, 8
    x = synth.activations(m, k, seed=1).cuda()
    for trial in range(6):
        qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=trial)
        w, sd, qzd = A.awq_repack_kmajor(qw.cuda()), s.cuda(), qz.cuda()
        first = A.awq_gemm(x, w, sd, qzd, 8, kernel=A.KERNEL_Q8).clone()
        torch.cuda.synchronize()
        assert device_status() == 0, f"trial {trial}"
        again = A.awq_gemm(x, w, sd, qzd, 8, kernel=A.KERNEL_Q8)
        assert torch.equal(first, again), f"trial {trial}"


def test_q8_rejects_what_it_cannot_take(A):
    from awq_b200 import synth, _lib
    qw, s, qz = [t.cuda() for t in synth.awq_linear_tensors(256, 256, 128, seed=0)]
    km = A.awq_repack_kmajor(qw)
    x = synth.activations(17, 256, seed=0).cuda()
    with pytest.raises(ValueError):            # more than 16 tokens
        A.awq_gemm(x, km, s, qz, 8, kernel=A.KERNEL_Q8)
    lib = _lib.load()
    assert lib.awq_b200_repack_kmajor_bytes(256, 256) == 256 * 256 // 2
    assert lib.awq_b200_repack_kmajor_bytes(256, 264) == 256 * 512 // 2   # padded to a whole slab
    assert lib.awq_b200_repack_kmajor_bytes(192, 256) == 0                # K % 128
    # scratch too small
    ws = torch.empty(1024, dtype=torch.uint8, device="cuda")
    out = torch.empty(1, 256, dtype=torch.float16, device="cuda")
    rc = lib.awq_b200_gemm(x.data_ptr(), km.data_ptr(), s.data_ptr(), qz.data_ptr(), None,
                           out.data_ptr(), 1, 256, 256, 128, A.KERNEL_Q8, ws.data_ptr(), 1024, None)
    assert rc == -5


def test_bounded_waits_give_up_and_the_context_survives(A):
    """A wait that nothing satisfies runs out after its limit, records its code in the status
    word and lets the kernel return; the status word is sticky until cleared; afterwards the
    GPU context is still usable."""
    from awq_b200 import synth, _lib
    lib = _lib.load()
    assert device_status() == 0
    assert lib.awq_b200_selftest_wait(2000, None) == 0
    torch.cuda.synchronize()
    assert device_status(clear=False) == 90       # the mbarrier wait gave up first
    assert device_status(clear=False) == 90       # sticky
    assert device_status(clear=True) == 90
    assert device_status() == 0                   # cleared
    run_case(A, 16, 1024, 512, seed=2, check_pack=False)
