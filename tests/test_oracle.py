"""The CPU oracle against vectors that do not come from this repository: vLLM's packer and
vLLM's Triton AWQ kernels (run by the Triton CPU interpreter, see tests/golden/make_golden.py),
the known word 0x75316420 and the moe_align_block_size docstring example."""
import numpy as np
import pytest

from oracle import awq_oracle as O

CASES = ["tiny", "ragged_m", "two_groups", "wide", "g64"]


def test_known_word(golden):
    assert golden["known_word"].view(np.uint32)[0, 0] == 0x75316420
    assert O.pack_awq(np.arange(8).reshape(1, 8)).view(np.uint32)[0, 0] == 0x75316420
    assert O.unpack_awq(np.array([[0x75316420]], dtype=np.uint32).view(np.int32)).tolist() == [
        list(range(8))]


@pytest.mark.parametrize("name", CASES)
def test_pack_unpack_bit_exact(golden, name):
    q = golden[f"{name}.nibbles"]
    z = golden[f"{name}.zero_nibbles"]
    assert np.array_equal(O.pack_awq(q), golden[f"{name}.qweight"])
    assert np.array_equal(O.pack_awq(z), golden[f"{name}.qzeros"])
    assert np.array_equal(O.unpack_awq(golden[f"{name}.qweight"]), q)
    assert np.array_equal(O.unpack_awq(golden[f"{name}.qzeros"]), z)


@pytest.mark.parametrize("name", CASES)
def test_dequantize_matches_reference_kernel_bit_exact(golden, name):
    g = int(golden[f"{name}.group"][0])
    w = O.dequantize_fp16(golden[f"{name}.qweight"], golden[f"{name}.scales"],
                          golden[f"{name}.qzeros"], g)
    assert np.array_equal(w.view(np.uint16), golden[f"{name}.w_fp16"].view(np.uint16))


@pytest.mark.parametrize("name", CASES)
def test_gemm_matches_reference_kernel(golden, name):
    """The reference Triton kernel accumulates in fp16 (awq_triton.py:134,216), the oracle in
    fp32: they agree to fp16-accumulation accuracy, not bit for bit."""
    g = int(golden[f"{name}.group"][0])
    y = O.awq_gemm_fp32(golden[f"{name}.x"], golden[f"{name}.qweight"], golden[f"{name}.scales"],
                        golden[f"{name}.qzeros"], g)
    ref = golden[f"{name}.y_fp16_triton"].astype(np.float32)
    assert O.rel_err(ref, y) < 1e-2


def test_moe_align_docstring_example(golden):
    ids = golden["align.topk_ids"]
    sorted_ids, expert_ids, post = O.moe_align_block_size(ids, int(golden["align.block"][0]),
                                                          int(golden["align.num_experts"][0]))
    assert post[0] == 16
    assert np.array_equal(sorted_ids[:16], golden["align.sorted_ids"])
    assert expert_ids[:4].tolist() == [0, 1, 2, 3]


def test_moe_align_properties():
    rng = np.random.default_rng(0)
    for t, k, e, blk in [(1, 8, 128, 16), (16, 8, 128, 16), (33, 2, 8, 4), (128, 8, 128, 16)]:
        ids = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.int32)
        s, eid, post = O.moe_align_block_size(ids, blk, e)
        n = t * k
        assert s.size == O.sorted_ids_capacity(n, e, blk)
        assert post[0] % blk == 0 and post[0] <= s.size
        real = s[s < n]
        assert sorted(real.tolist()) == list(range(n))          # a permutation of all pairs
        flat = ids.reshape(-1)
        for b in range(post[0] // blk):
            seg = s[b * blk:(b + 1) * blk]
            seg = seg[seg < n]
            assert np.all(flat[seg] == eid[b])                   # block is single-expert
            assert np.all(np.diff(seg) > 0)                      # ascending = stable
        assert np.all(eid[post[0] // blk:] == -1)


def test_moe_align_expert_map():
    ids = np.array([[0, 1], [1, 2], [2, 3]], dtype=np.int32)
    emap = np.array([-1, 0, -1, 1], dtype=np.int32)
    s, eid, post = O.moe_align_block_size(ids, 2, 4, emap)
    assert post[0] == 4
    assert s[:4].tolist() == [1, 2, 5, 6]
    assert eid[:2].tolist() == [0, 1]


def test_topk_softmax():
    rng = np.random.default_rng(1)
    g = rng.standard_normal((7, 128)).astype(np.float32)
    w, ids, tok = O.topk_softmax(g, 8, True)
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    for t in range(7):
        assert ids[t].tolist() == np.argsort(-g[t], kind="stable")[:8].tolist()
    assert tok[3, 2] == 2 * 7 + 3
    g[0, 5] = g[0, 9] = 10.0   # tie -> lower id first
    _, ids, _ = O.topk_softmax(g, 2, False)
    assert ids[0].tolist() == [5, 9]


def test_fused_experts_against_dense_loop():
    import torch
    rng = np.random.default_rng(2)
    e, h, i, t, k = 4, 256, 128, 5, 2
    def mk(r, c):
        return O.pack_awq(rng.integers(0, 16, (r, c)))
    w13_q = np.stack([mk(h, 2 * i) for _ in range(e)])
    w13_z = np.stack([mk(h // 128, 2 * i) for _ in range(e)])
    w13_s = rng.uniform(0.002, 0.02, (e, h // 128, 2 * i)).astype(np.float16)
    w2_q = np.stack([mk(i, h) for _ in range(e)])
    w2_z = np.stack([mk(i // 128, h) for _ in range(e)])
    w2_s = rng.uniform(0.002, 0.02, (e, i // 128, h)).astype(np.float16)
    x = rng.standard_normal((t, h)).astype(np.float16)
    w, ids, _ = O.topk_softmax(rng.standard_normal((t, e)).astype(np.float32), k, True)
    y = O.fused_experts_fp32(x, w13_q, w13_s, w13_z, w2_q, w2_s, w2_z, w, ids,
                             round_intermediate=False)
    ref = np.zeros((t, h), dtype=np.float64)
    for tt in range(t):
        for s in range(k):
            ee = ids[tt, s]
            a = x[tt].astype(np.float64) @ O.dequantize_fp32(w13_q[ee], w13_s[ee], w13_z[ee])
            act = a[:i] / (1 + np.exp(-a[:i])) * a[i:]
            ref[tt] += w[tt, s] * (act @ O.dequantize_fp32(w2_q[ee], w2_s[ee], w2_z[ee]))
    assert O.rel_err(y, ref) < 1e-4


def test_torch_form_of_the_oracle_matches_numpy_form(golden):
    import torch
    for name in CASES:
        g = int(golden[f"{name}.group"][0])
        a = [golden[f"{name}.{k}"] for k in ("x", "qweight", "scales", "qzeros")]
        y_np = O.awq_gemm_fp32(*a, g)
        y_t = O.awq_gemm_fp32_torch(*[torch.from_numpy(v) for v in a], g).numpy()
        assert np.allclose(y_np, y_t, rtol=1e-5, atol=1e-5)


def test_pack_kmajor_layout():
    """The K-major repack permutes the unpacked nibbles: tile (slab, group) = 256 rows of 64 bytes,
    row r = column 256 * slab + r, nibble j of the row = k 128 * group + j; columns past N zero."""
    rng = np.random.default_rng(5)
    k, n = 256, 264                     # two groups, one full slab and 8 columns of a second
    q = rng.integers(0, 16, size=(k, n), dtype=np.int64)
    packed = O.pack_awq(q)
    km = O.pack_kmajor(packed).reshape(2, 2, 256, 64)        # slab, group, row, byte
    for slab, g, r, b in [(0, 0, 0, 0), (0, 1, 255, 63), (1, 0, 7, 10), (1, 1, 3, 31)]:
        col = 256 * slab + r
        lo, hi = q[128 * g + 2 * b, col], q[128 * g + 2 * b + 1, col]
        assert km[slab, g, r, b] == (lo | (hi << 4))
    assert not km[1, :, 8:, :].any()    # padding columns
    assert km.size == 2 * 2 * 256 * 64


def test_wna16_layout_against_vllm_converter():
    """The MoE WNA16 byte layout as vLLM's own weight-loader converter produces it
    (tests/golden/make_wna16_golden.py), both directions, bit-exact."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                             "wna16_golden.npz"))
    for name in ("small", "wide", "g64"):
        w = O.awq_to_wna16_qweight(g[f"{name}.qweight"])
        z = O.awq_to_wna16_qzeros(g[f"{name}.qzeros"])
        assert np.array_equal(w, g[f"{name}.wna16_qweight"])
        assert np.array_equal(z, g[f"{name}.wna16_qzeros"])
        assert np.array_equal(g[f"{name}.wna16_scales"], g[f"{name}.scales"].T)
        assert np.array_equal(O.wna16_to_awq_qweight(w), g[f"{name}.qweight"])
        assert np.array_equal(O.wna16_to_awq_qzeros(z), g[f"{name}.qzeros"])


def test_fixed_point_model_of_the_kmajor_kernel_stays_below_fp16_rounding():
    """What rewriting the activations as 24-bit fixed point per token may cost: against the fp32
    reference the model is off by well under fp16's own rounding of the output, also when one
    element of a token is a thousand times larger than the rest."""
    from awq_b200 import synth
    k, n, m = 1024, 256, 16
    qw, s, qz = synth.awq_linear_tensors(k, n, 128, seed=3)
    x = synth.activations(m, k, seed=4).numpy().astype(np.float32)
    x[3, 17] = 1000.0           # an outlier sets the token's scale
    x[5] = 0.0                  # an all-zero token
    x16 = x.astype(np.float16)
    ref = O.awq_gemm_fp32(x16, qw.numpy(), s.numpy(), qz.numpy(), 128)
    got = O.awq_gemm_fixed_point_model(x16, qw.numpy(), s.numpy(), qz.numpy(), 128)
    assert np.isfinite(got).all() and not got[5].any()
    assert O.rel_err(got, ref) < 1e-4
    for t in range(m):          # per token too: the outlier row keeps its accuracy
        denom = np.abs(ref[t]).max()
        if denom > 0:
            assert np.abs(got[t] - ref[t]).max() / denom < 2e-4
