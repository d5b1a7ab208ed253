"""The decode-layout copy of qweight and the streaming kernel that reads it: the copy is
bit-exact against its definition, the kernel agrees with the CPU oracle and, bit for bit, with
the same kernel on the checkpoint layout."""
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


def decode_layout(qweight: np.ndarray) -> np.ndarray:
    """[K, W] int32 -> [K/4, W, 4] uint32: for rows (k..k+3) of one word column the low and
    high halfwords of the pairs (k, k+1) and (k+2, k+3), low row in the low half."""
    k, w = qweight.shape
    q = qweight.view(np.uint32).reshape(k // 4, 4, w)
    lo = lambda a, b: (a & 0xFFFF) | ((b & 0xFFFF) << 16)  # noqa: E731
    hi = lambda a, b: (a >> 16) | (b & 0xFFFF0000)  # noqa: E731
    return np.stack([lo(q[:, 0], q[:, 1]), hi(q[:, 0], q[:, 1]),
                     lo(q[:, 2], q[:, 3]), hi(q[:, 2], q[:, 3])], axis=-1)


@pytest.mark.parametrize("k,n", [(4, 8), (128, 32), (256, 288), (1024, 512), (8192, 1024)])
def test_repack_is_bit_exact(A, k, n):
    rng = np.random.default_rng(k + n)
    qw = torch.from_numpy(rng.integers(-2**31, 2**31, size=(k, n // 8), dtype=np.int64)
                          .astype(np.int32))
    got = A.awq_repack(qw.cuda()).cpu().numpy().view(np.uint32).reshape(k // 4, n // 8, 4)
    assert np.array_equal(got, decode_layout(qw.numpy()))


def test_repack_rejects_bad_input(A):
    with pytest.raises(ValueError):
        A.awq_repack(torch.zeros((6, 4), dtype=torch.int32, device="cuda"))
    with pytest.raises((TypeError, ValueError)):
        A.awq_repack(torch.zeros((8, 4), dtype=torch.int64, device="cuda"))
    assert A.awq_repack(torch.zeros((0, 4), dtype=torch.int32, device="cuda")).shape == (0, 4)


@pytest.mark.parametrize("m,k,n", [(1, 128, 32), (1, 512, 256), (3, 384, 288), (8, 1024, 512),
                                   (5, 8192, 1024), (8, 3712, 8192), (2, 29568, 1024)])
def test_decode_layout_gemm_vs_oracle_and_checkpoint_layout(A, m, k, n):
    from awq_b200 import synth
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=m + k + n)
    x = synth.activations(m, k, seed=m)
    b = torch.randn(n, generator=torch.Generator().manual_seed(m)).half()
    dq, ds, dz, dx, db = (t.cuda() for t in (qw, s, qz, x, b))
    rp = A.awq_repack(dq)
    y = A.awq_gemm(dx, rp, ds, dz, 8, bias=db, kernel=A.KERNEL_STREAM_RP)
    y_plain = A.awq_gemm(dx, dq, ds, dz, 8, bias=db, kernel=A.KERNEL_STREAM)
    assert torch.equal(y, y_plain)
    ref = O.awq_gemm_fp32(x.numpy(), qw.numpy(), s.numpy(), qz.numpy(), 128)
    ref = ref + b.numpy().astype(np.float32)
    y = y.cpu().numpy()
    assert O.rel_err(y, ref) < TOL
    assert O.elementwise_ok(y, ref, TOL)


def test_decode_layout_kernel_rejects_unsupported_shapes(A):
    from awq_b200 import synth
    qw, s, qz = (t.cuda() for t in synth.awq_linear_tensors(256, 256, 128, seed=1))
    with pytest.raises(ValueError):   # more tokens than the kernel serves
        A.awq_gemm(synth.activations(9, 256).cuda(), qw, s, qz, 8, kernel=A.KERNEL_STREAM_RP)
    qw, s, qz = (t.cuda() for t in synth.awq_linear_tensors(256, 256, 64, seed=1))
    with pytest.raises(ValueError):   # group size other than 128
        A.awq_gemm(synth.activations(1, 256).cuda(), qw, s, qz, 8, kernel=A.KERNEL_STREAM_RP)


def test_linear_method_with_decode_copy(A):
    from awq_b200 import synth
    k, n = 1024, 768
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=21)
    layers = []
    for repack in (False, True):
        method = A.AWQLinearMethod(A.AWQConfig(group_size=128, repack_decode=repack))
        layer = A.AWQLinear()
        method.create_weights(layer, k, [n], k, n, torch.float16)
        layer.qweight.data.copy_(qw)
        layer.scales.data.copy_(s)
        layer.qzeros.data.copy_(qz)
        method.process_weights_after_loading(layer)
        layers.append((method, layer))
    assert layers[0][1].qweight_decode is None
    assert layers[1][1].qweight_decode is not None
    for m in (1, 8, 9, 40):     # 9 and 40 leave the decode copy unused
        x = synth.activations(m, k, seed=m).cuda()
        y0 = layers[0][0].apply(layers[0][1], x)
        y1 = layers[1][0].apply(layers[1][1], x)
        ref = O.awq_gemm_fp32(x.cpu().numpy(), qw.numpy(), s.numpy(), qz.numpy(), 128)
        assert O.rel_err(y1.cpu().numpy(), ref) < TOL
        if m > 8:
            assert torch.equal(y0, y1)
