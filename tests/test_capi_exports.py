"""The C-ABI library loads and exports every symbol include/awq_b200.h declares; host-side
validation paths that need no GPU return the documented codes."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "awq_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(awq_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for n in ["awq_b200_gemm", "awq_b200_dequantize", "awq_b200_topk_softmax",
              "awq_b200_moe_align_block_size", "awq_b200_moe_experts", "awq_b200_strerror"]:
        assert n in names


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in awq_b200.h but not exported"


def test_python_prototypes_cover_the_header(built_library):
    from awq_b200 import _lib
    assert sorted(_lib.PROTOTYPES) == declared_symbols()
    lib = _lib.load()
    assert lib.awq_b200_version().decode() == "0.1"
    assert _lib.strerror(0) == "ok"
    assert "NULL" in _lib.strerror(-1)
    assert "unknown" in _lib.strerror(-1234)


def test_host_side_validation_without_gpu(built_library):
    """Argument checks run before any CUDA call, so they are testable on a CPU-only box."""
    from awq_b200 import _lib
    lib = _lib.load()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 255) & ~255
    # NULL pointer
    assert lib.awq_b200_gemm(None, p, p, p, None, p, 1, 8, 128, 128, 0, None, 0, None) == -1
    # N not a multiple of 8
    assert lib.awq_b200_gemm(p, p, p, p, None, p, 1, 12, 128, 128, 0, None, 0, None) == -2
    # K not a multiple of the group
    assert lib.awq_b200_gemm(p, p, p, p, None, p, 1, 8, 192, 128, 0, None, 0, None) == -2
    # group not a multiple of 8
    assert lib.awq_b200_dequantize(p, p, p, p, 100, 8, 100, None) == -4
    # misaligned pointer
    assert lib.awq_b200_gemm(p + 4, p, p, p, None, p, 1, 8, 128, 128, 0, None, 0, None) == -3
    # M == 0 is a no-op
    assert lib.awq_b200_gemm(None, None, None, None, None, None, 0, 8, 128, 128, 0, None, 0,
                             None) == 0
    # capacity formula (fused_moe/moe_align_block_size.py:74-80)
    assert lib.awq_b200_moe_sorted_capacity(8, 128, 16) == 128
    assert lib.awq_b200_moe_sorted_capacity(1024, 128, 16) == 1024 + 128 * 15
    # router limits
    assert lib.awq_b200_topk_softmax(p, 0, 4, 2048, 8, 1, p, p, p, None) == -9
    assert lib.awq_b200_topk_softmax(p, 0, 4, 8, 9, 1, p, p, p, None) == -2
    # sorted_ids too small
    assert lib.awq_b200_moe_align_block_size(p, 4, 2, 8, 4, None, p, 3, p, p, None) == -5


def test_moe_scratch_check_follows_sorted_capacity(built_library):
    """The expert entry points lay their scratch out for round_up(sorted_capacity, block) rows.
    Under expert parallelism the caller passes the local expert count but a permutation (and
    sorted_capacity) built for the global one: the size check must use that capacity, and must
    refuse before anything is launched (no GPU is needed to see the refusal)."""
    from awq_b200 import _lib
    lib = _lib.load()
    buf = (ctypes.c_char * 4096)()
    p = (ctypes.addressof(buf) + 255) & ~255
    T, topk, e_local, e_global, H, I, block = 320, 8, 16, 128, 2048, 768, 16
    cap = lib.awq_b200_moe_sorted_capacity(T * topk, e_global, block)
    assert cap == T * topk + e_global * (block - 1)
    limit = lib.awq_b200_moe_static_scratch_bytes()
    rows = -(-cap // block) * block
    need = -(-rows * I * 2 // 256) * 256 + -(-T * topk * H * 2 // 256) * 256
    # the hole this closes: the layout for the local expert count's capacity fits the 16 MiB,
    # the layout for the capacity actually passed does not
    cap_local = lib.awq_b200_moe_sorted_capacity(T * topk, e_local, block)
    need_local = -(-cap_local // block) * block * I * 2 + T * topk * H * 2
    assert need_local <= limit < need
    args = [p] * 7 + [p] * 4 + [p] + [T, topk, e_local, H, I, 128, block, 1]
    assert lib.awq_b200_moe_experts_static(*args, cap, None) == -9
    assert lib.awq_b200_moe_experts(*args, cap, p, limit, None) == -5
    # a capacity far above the minimum is legal for the permutation but not for a small buffer
    big = 4 * cap
    assert lib.awq_b200_moe_experts_static(*args, big, None) == -9
    assert lib.awq_b200_moe_experts(*args, big, p, need, None) == -5
    # and the text of the new code
    assert "scratch" in _lib.strerror(-10)


def test_ops_reject_cpu_tensors(built_library):
    import torch
    import awq_b200
    q = torch.zeros(128, 1, dtype=torch.int32)
    s = torch.zeros(1, 8, dtype=torch.float16)
    x = torch.zeros(1, 128, dtype=torch.float16)
    with pytest.raises(ValueError, match="no CPU path"):
        awq_b200.awq_gemm(x, q, s, q[:1], 8)
    with pytest.raises(ValueError, match="no CPU path"):
        awq_b200.awq_dequantize(q, s, q[:1], 0, 0, 0)


def test_linear_method_weight_contract(built_library):
    import torch
    from awq_b200 import AWQConfig, AWQLinear, AWQLinearMethod
    m = AWQLinearMethod(AWQConfig(group_size=128))
    layer = AWQLinear()
    m.create_weights(layer, 256, [64, 64], 256, 128, torch.float16, device="cpu")
    assert layer.qweight.shape == (256, 16) and layer.qweight.dtype == torch.int32
    assert layer.qzeros.shape == (2, 16) and layer.scales.shape == (2, 128)
    with pytest.raises(ValueError, match="input size is not aligned"):
        m.create_weights(AWQLinear(), 200, [64], 200, 64, torch.float16, device="cpu")
    with pytest.raises(ValueError, match="output size is not aligned"):
        m.create_weights(AWQLinear(), 256, [60], 256, 60, torch.float16, device="cpu")
    with pytest.raises(ValueError):
        AWQConfig(weight_bits=8)


def test_missing_library_fails_loudly(monkeypatch, built_library):
    from awq_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libawq_b200.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()


def test_repack_and_block_size_host_logic(built_library):
    """Host-side checks of the decode-layout repack and the MoE row-block choice (no GPU)."""
    from awq_b200 import _lib
    lib = _lib.load()
    buf = (ctypes.c_char * 4096)()
    p = (ctypes.addressof(buf) + 255) & ~255
    assert lib.awq_b200_repack_qweight(None, p, 8, 8, None) == -1
    assert lib.awq_b200_repack_qweight(p, p + 1024, 6, 8, None) == -2      # K % 4
    assert lib.awq_b200_repack_qweight(p, p + 1024, 8, 12, None) == -2     # N % 8
    assert lib.awq_b200_repack_qweight(p + 4, p + 1024, 8, 8, None) == -3  # alignment
    # Qwen3-30B-A3B shapes: 8-row blocks up to eight rows per expert on average, 16-row blocks up
    # to 36, grouped tcgen05 GEMMs (128) from there on
    e, h, i, k = 128, 2048, 768, 8
    assert [lib.awq_b200_moe_block_size(t, k, e, h, i, 128) for t in (1, 16, 128, 129, 512, 575, 576,
                                                                     4096)] == \
        [8, 8, 8, 16, 16, 16, 128, 128]
    # shapes the grouped tcgen05 kernels do not tile stay on the streaming kernels
    assert lib.awq_b200_moe_block_size(4096, k, e, 2048 + 128, i, 128) == 16


def test_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: one JSON line with the keys the contract names."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True,
                         timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config",
                "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] in ("port", "reference")
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0


def test_validation_of_the_newer_entry_points_without_gpu(built_library):
    """Exchange, layout conversion and the direct MoE mode refuse bad arguments before any CUDA
    call."""
    from awq_b200 import _lib
    lib = _lib.load()
    buf = (ctypes.c_char * 8192)()
    p = (ctypes.addressof(buf) + 255) & ~255
    regions = (ctypes.c_void_p * 2)(p, p)
    # all-reduce: rank count, rank, offsets, sizes, NULLs, alignment
    assert lib.awq_b200_allreduce(regions, 0, 9, 4096, p, 32, p, 0, None) == -2
    assert lib.awq_b200_allreduce(regions, 2, 2, 4096, p, 32, p, 0, None) == -2
    assert lib.awq_b200_allreduce(regions, 0, 2, 16, p, 32, p, 0, None) == -2      # inside the flags
    assert lib.awq_b200_allreduce(regions, 0, 2, 4096, p, 24, p, 0, None) == -2    # not 16-byte units
    assert lib.awq_b200_allreduce(None, 0, 2, 4096, p, 32, p, 0, None) == -1
    assert lib.awq_b200_allreduce(regions, 0, 2, 4096, p, 32, None, 0, None) == -1
    assert lib.awq_b200_allreduce(regions, 0, 2, 4096, p, 0, p, 0, None) == 0      # nothing to do
    odd = (ctypes.c_void_p * 2)(p, p + 8)
    assert lib.awq_b200_allreduce(odd, 0, 2, 4096, p, 32, p, 0, None) == -3
    hole = (ctypes.c_void_p * 2)(p, None)
    assert lib.awq_b200_allreduce(hole, 0, 2, 4096, p, 32, p, 0, None) == -1
    # peer regions
    out = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    assert lib.awq_b200_peer_region_create(100, ctypes.byref(out), handle) == -2   # below the flag area
    assert lib.awq_b200_peer_region_create(8192, None, handle) == -1
    assert lib.awq_b200_peer_region_open(None, ctypes.byref(out)) == -1
    assert lib.awq_b200_peer_region_close(None) == -1
    # MoE WNA16 layout conversion
    assert lib.awq_b200_wna16_to_awq(p, p, p, p, p, p, 1, 12, 128, 128, None) == -2   # N % 8
    assert lib.awq_b200_wna16_to_awq(p, p, p, p, p, p, 1, 8, 192, 128, None) == -2    # K % group
    assert lib.awq_b200_wna16_to_awq(p, p, None, p, p, p, 1, 8, 128, 128, None) == -1
    # direct MoE mode: block 8 only, not with an expert map, bounded pair count, exact capacity
    T, topk, E, H, I = 2, 8, 128, 2048, 768
    base = [p] * 7 + [p, None, p, None, p]
    tail = lambda block, flags, cap: [T, topk, E, H, I, 128, block, flags, cap, p, 1 << 30, None]  # noqa: E731
    assert lib.awq_b200_moe_experts(*base, *tail(16, 4, T * topk * 8)) == -2
    assert lib.awq_b200_moe_experts(*base, *tail(8, 5, T * topk * 8)) == -2
    assert lib.awq_b200_moe_experts(*base, *tail(8, 4, T * topk * 8 + 8)) == -5
    many = [p] * 7 + [p, None, p, None, p] + [16, topk, E, H, I, 128, 8, 4, 16 * topk * 8, p, 1 << 30, None]
    assert lib.awq_b200_moe_experts(*many) == -2                                   # 128 pairs > 64
    # without the flag the permutation tables are required
    assert lib.awq_b200_moe_experts(*base, *tail(8, 0, T * topk * 8)) == -1
