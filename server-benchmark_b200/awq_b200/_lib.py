"""ctypes binding of libawq_b200.so (the C ABI declared in include/awq_b200.h).

The library is the only compute path: if it is missing this module raises, there is no
Python or CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libawq_b200.so")

OK = 0
KERNEL_AUTO = 0
KERNEL_GENERIC = 1
KERNEL_STREAM = 2
KERNEL_TCGEN05 = 3
KERNEL_STREAM_EXACT = 4
KERNEL_TS = 5
KERNEL_TS_EXACT = 6
KERNEL_WT = 7
KERNEL_STREAM_RP = 8
KERNEL_Q8 = 9

# name -> (restype, argtypes); kept in step with include/awq_b200.h
PROTOTYPES = {
    "awq_b200_strerror": (c_char_p, [c_int]),
    "awq_b200_version": (c_char_p, []),
    "awq_b200_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                    c_void_p]),
    "awq_b200_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "awq_b200_repack_qweight": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "awq_b200_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                              c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "awq_b200_device_status": (c_int, [POINTER(c_int)]),
    "awq_b200_device_status_clear": (c_int, [POINTER(c_int)]),
    "awq_b200_set_wait_limit": (None, [c_uint]),
    "awq_b200_selftest_wait": (c_int, [c_uint, c_void_p]),
    "awq_b200_repack_kmajor_bytes": (c_size_t, [c_int, c_int]),
    "awq_b200_repack_kmajor": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "awq_b200_allreduce": (c_int, [c_void_p, c_int, c_int, c_size_t, c_void_p, c_size_t, c_void_p,
                                   c_int, c_void_p]),
    "awq_b200_peer_region_create": (c_int, [c_size_t, c_void_p, c_void_p]),
    "awq_b200_peer_region_open": (c_int, [c_void_p, c_void_p]),
    "awq_b200_peer_region_close": (c_int, [c_void_p]),
    "awq_b200_peer_region_destroy": (c_int, [c_void_p]),
    "awq_b200_wna16_to_awq": (c_int, [c_void_p] * 6 + [c_int] * 4 + [c_void_p]),
    "awq_b200_topk_softmax": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                      c_void_p, c_void_p, c_void_p]),
    "awq_b200_moe_sorted_capacity": (c_int64, [c_int64, c_int, c_int]),
    "awq_b200_moe_align_block_size": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                              c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "awq_b200_moe_block_size": (c_int, [c_int] * 6),
    "awq_b200_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "awq_b200_moe_experts": (c_int, [c_void_p] * 7 + [c_void_p] * 4 + [c_void_p] +
                             [c_int] * 8 + [c_int64, c_void_p, c_size_t, c_void_p]),
    "awq_b200_moe_static_scratch_bytes": (c_size_t, []),
    "awq_b200_moe_experts_static": (c_int, [c_void_p] * 7 + [c_void_p] * 4 + [c_void_p] +
                                    [c_int] * 8 + [c_int64, c_void_p]),
}

_lib = None


class AwqB200Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed: {text} (code {code})")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the shared library once and attach prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python server-benchmark_b200/build.py` "
            "(the CUDA library is the only compute path, there is no fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().awq_b200_strerror(code).decode()


def check(fn: str, code: int) -> None:
    """Map a status code to the exception the reference raises in the same situation:
    shape / group / alignment problems are ValueError (vLLM raises ValueError for bad
    partitioning, quantization/awq.py:198-211), the rest RuntimeError."""
    if code == OK:
        return
    text = strerror(code)
    if code in (-1, -2, -3, -4, -9):
        raise ValueError(f"{fn}: {text} (code {code})")
    raise AwqB200Error(fn, code, text)
