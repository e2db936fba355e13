"""ctypes binding of ``libvqg_b200.so`` (the C ABI declared in include/vqg.h).

Loading fails loudly: there is no Python or CPU substitute for the CUDA library.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_longlong, c_size_t, c_uint, c_ulonglong, c_void_p, POINTER

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libvqg_b200.so")

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_LAUNCH, ERR_DEVICE_TIMEOUT, ERR_NO_DEVICE, ERR_TOO_LARGE, ERR_NO_MEMORY = range(9)
LAYOUT_BL, LAYOUT_REF = 0, 1
IDX_PACKED12 = 12      # idx_bytes value: two 12-bit indices in three bytes
PATH_AUTO, PATH_GENERIC, PATH_DECODE, PATH_TENSOR, PATH_TWO_PHASE, PATH_TENSOR_PAIR, PATH_TENSOR_TS, PATH_SMALL_TS = range(8)
PATHS = {"auto": PATH_AUTO, "generic": PATH_GENERIC, "decode": PATH_DECODE, "tensor": PATH_TENSOR,
         "two_phase": PATH_TWO_PHASE, "tensor_pair": PATH_TENSOR_PAIR, "tensor_ts": PATH_TENSOR_TS, "small_ts": PATH_SMALL_TS}

# name -> (restype, argtypes); mirrors include/vqg.h one to one
SIGNATURES = {
    "vqg_version": (c_int, []),
    "vqg_status_string": (c_char_p, [c_int]),
    "vqg_workspace_bytes": (c_size_t, [c_int] * 9),
    "vqg_workspace_counter_bytes": (c_size_t, []),
    "vqg_gemm": (c_int, [c_void_p] * 4 + [c_int] * 8 + [c_void_p, c_size_t, c_void_p]),
    "vqg_gemm_path": (c_int, [c_void_p] * 4 + [c_int] * 9 + [c_void_p, c_size_t, c_void_p]),
    "vqg_dequant": (c_int, [c_void_p] * 3 + [c_int] * 7 + [c_void_p]),
    "vqg_dense_gemm": (c_int, [c_void_p] * 3 + [c_int] * 4 + [c_void_p, c_size_t, c_void_p]),
    "vqg_dense_workspace_bytes": (c_size_t, [c_int] * 4),
    "vqg_gemm_sharded": (c_int, [c_void_p] * 3 + [POINTER(c_void_p), c_int, c_int] + [c_int] * 7
                         + [c_void_p, c_size_t, c_void_p]),
    "vqg_gemm_sharded_mc": (c_int, [c_void_p] * 3 + [POINTER(c_void_p), c_void_p, c_int, c_int] + [c_int] * 7
                            + [c_void_p, c_size_t, c_void_p]),
    "vqg_gemm_sharded_cols": (c_int, [c_void_p] * 3 + [POINTER(c_void_p), c_void_p, c_int, c_int] + [c_int] * 7
                              + [c_longlong, c_longlong, c_void_p, c_size_t, c_void_p]),
    "vqg_rank_barrier": (c_int, [POINTER(c_void_p), c_int, c_int, c_uint, c_longlong, c_void_p]),
    "vqg_residual_workspace_bytes": (c_size_t, [c_int] * 8),
    "vqg_gemm_residual": (c_int, [c_void_p] * 4 + [c_int] * 8 + [c_void_p, c_size_t, c_void_p]),
    "vqg_dequant_residual": (c_int, [c_void_p] * 3 + [c_int] * 7 + [c_void_p]),
    "vqg_swiglu_workspace_bytes": (c_size_t, [c_int] * 7),
    "vqg_gemm_swiglu": (c_int, [c_void_p] * 4 + [c_int] * 7 + [c_void_p, c_size_t, c_void_p]),
    "vqg_rowparallel_workspace_bytes": (c_size_t, [c_int] * 7),
    "vqg_gemm_rowparallel": (c_int, [c_void_p] * 3 + [POINTER(c_void_p)] + [c_int] * 8 + [c_void_p, c_size_t, c_void_p]),
    "vqg_reduce_slots": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_void_p]),
    "vqg_auto_path": (c_int, [c_int] * 8),
    "vqg_selftest_bounded_wait": (c_int, [c_longlong, c_void_p]),
    "vqg_quantize_assign": (c_int, [c_void_p] * 3 + [c_int] * 6 + [c_void_p]),
    "vqg_quantize_workspace_bytes": (c_size_t, [c_int] * 4),
    "vqg_quantize_update": (c_int, [c_void_p] * 4 + [c_size_t] + [c_int] * 6 + [c_void_p]),
    "vqg_pack12": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p]),
    "vqg_unpack12": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p]),
    "vqg_gemm_small_batch_noalloc": (c_int, [c_void_p] * 4 + [c_int] * 7 + [c_void_p]),
    "vqg_device_status": (c_int, [POINTER(c_int)]),
    "vqg_launch_count": (c_ulonglong, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Returns the loaded library; raises if it has not been built (python -m vq_gemm_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python compile_kernels.py build_ext --inplace` "
            "(or `python -m vq_gemm_b200.build`). There is no fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library is stale
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(code: int) -> str:
    return load().vqg_status_string(code).decode()


def check(code: int, what: str) -> None:
    if code != OK:
        raise RuntimeError(f"{what}: {status_string(code)} (status {code})")
