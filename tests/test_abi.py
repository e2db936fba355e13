"""The C-ABI library loads on a machine without a GPU, exports every symbol the header declares,
and rejects bad arguments before touching CUDA.  No compute calls here."""
import ctypes
import os
import re

import pytest

from vq_gemm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from vq_gemm_b200.build import build
    build()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "vqg.h")).read()
    return sorted(set(re.findall(r"VQG_API[^;(]*?\b(vqg_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = _declared()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/vqg.h but not exported"
    assert sorted(_lib.SIGNATURES) == names


def test_no_torch_or_python_dependency():
    import subprocess
    out = subprocess.run(["ldd", _lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "torch" not in out and "python" not in out and "libcuda.so" not in out


def test_status_strings(lib):
    seen = set()
    for code in range(8):
        s = _lib.status_string(code)
        assert s and s != "unknown status"
        seen.add(s)
    assert len(seen) == 8
    assert _lib.status_string(99) == "unknown status"
    assert lib.vqg_version() >= 100


def test_workspace_sizes(lib):
    cb = lib.vqg_workspace_counter_bytes()
    # K <= 4096 decode needs no scratch; K = 8192 splits K in two chunks of fp32 partials
    assert lib.vqg_workspace_bytes(1, 11008, 4096, 4, 256, 1, 128, 0, 0) == 0
    assert lib.vqg_workspace_bytes(16, 8192, 8192, 8, 4096, 2, 0, 0, _lib.PATH_DECODE) == cb + 2 * 16 * 8192 * 4
    # the small-batch tensor-memory kernel (what AUTO picks for 4 < M <= 128) keeps per-tile partial sums
    assert lib.vqg_workspace_bytes(16, 8192, 8192, 8, 4096, 2, 0, 0, _lib.PATH_SMALL_TS) > cb
    assert lib.vqg_workspace_bytes(16, 8192, 8192 + 64, 8, 4096, 2, 0, 0, _lib.PATH_SMALL_TS) == 0   # K % 128
    # two-phase: one fp16 copy of the dequantised weights
    assert lib.vqg_workspace_bytes(256, 512, 256, 4, 256, 1, 128, 0, _lib.PATH_TWO_PHASE) == cb + 512 * 256 * 2
    assert lib.vqg_workspace_bytes(0, 0, 0, 4, 256, 1, 0, 0, 0) == 0
    assert lib.vqg_dense_workspace_bytes(128, 256, 64, 1) == cb + 256 * 64 * 2
    assert lib.vqg_dense_workspace_bytes(128, 256, 64, 0) == 0


def test_bad_arguments_are_rejected_without_cuda(lib):
    p = ctypes.c_void_p(4096)
    null = None
    call = lib.vqg_gemm
    # negative size, unknown layout, null pointers, K not a multiple of v, index width vs C
    assert call(p, p, p, p, -1, 8, 8, 4, 256, 1, 0, 0, null, 0, null) == _lib.ERR_BAD_ARG
    assert call(p, p, p, p, 1, 8, 8, 4, 256, 1, 0, 7, null, 0, null) == _lib.ERR_BAD_ARG
    assert call(null, p, p, p, 1, 8, 8, 4, 256, 1, 0, 0, null, 0, null) == _lib.ERR_BAD_ARG
    assert call(p, p, p, null, 1, 8, 8, 4, 256, 1, 0, 0, null, 0, null) == _lib.ERR_BAD_ARG
    assert call(p, p, p, p, 1, 8, 10, 4, 256, 1, 0, 0, null, 0, null) == _lib.ERR_BAD_ARG
    assert call(p, p, p, p, 1, 8, 8, 4, 4096, 1, 0, 0, null, 0, null) == _lib.ERR_BAD_ARG
    assert call(p, p, p, p, 1, 8, 8, 4, 256, 3, 0, 0, null, 0, null) == _lib.ERR_UNSUPPORTED
    # reference format is v=2, C=256, uint8 only
    assert call(p, p, p, p, 1, 8, 8, 4, 256, 1, 0, 1, null, 0, null) == _lib.ERR_UNSUPPORTED
    # empty problems succeed without a launch
    assert call(p, p, p, p, 0, 8, 8, 4, 256, 1, 0, 0, null, 0, null) == _lib.OK
    assert call(p, p, p, p, 4, 0, 8, 4, 256, 1, 0, 0, null, 0, null) == _lib.OK
    assert lib.vqg_dequant(p, p, p, 0, 8, 4, 256, 1, 0, 0, null) == _lib.OK
    assert lib.vqg_dequant(null, p, p, 8, 8, 4, 256, 1, 0, 0, null) == _lib.ERR_BAD_ARG
    # misaligned pointers are refused with a status code, never handed to a kernel: 2-byte indices at an odd
    # address, a codebook or an output that is not 16-byte aligned
    odd = ctypes.c_void_p(4097)
    off8 = ctypes.c_void_p(4096 + 8)
    assert lib.vqg_dequant(odd, p, p, 8, 8, 4, 300, 2, 0, 0, null) == _lib.ERR_BAD_ARG
    assert lib.vqg_dequant(p, off8, p, 8, 8, 8, 256, 1, 0, 0, null) == _lib.ERR_BAD_ARG
    assert lib.vqg_dequant(p, p, off8, 8, 8, 8, 256, 1, 0, 0, null) == _lib.ERR_BAD_ARG
    # packed 12-bit indices: whole pairs per row, at most 4096 entries; only the plain product and dequant take them
    PK = _lib.IDX_PACKED12
    assert call(p, p, p, p, 1, 8, 24, 8, 4096, PK, 0, 0, null, 0, null) == _lib.ERR_BAD_ARG       # K/v = 3 is odd
    assert call(p, p, p, p, 1, 8, 32, 8, 5000, PK, 0, 0, null, 0, null) == _lib.ERR_BAD_ARG
    assert call(p, p, p, p, 1, 8, 32, 8, 4096, PK, 0, 1, null, 0, null) == _lib.ERR_UNSUPPORTED   # not in the reference's format
    assert lib.vqg_dequant(p, p, p, 8, 24, 8, 4096, PK, 0, 0, null) == _lib.ERR_BAD_ARG
    assert lib.vqg_gemm_swiglu(p, p, p, p, 1, 8, 32, 8, 4096, PK, 0, null, 0, null) == _lib.ERR_UNSUPPORTED
    assert lib.vqg_device_status(None) == _lib.ERR_BAD_ARG
    arr = (ctypes.c_void_p * 2)(4096, 8192)
    assert lib.vqg_gemm_sharded(p, p, p, arr, 2, 2, 1, 8, 8, 4, 256, 1, 0, null, 0, null) == _lib.ERR_BAD_ARG
    assert lib.vqg_gemm_sharded(p, p, p, arr, 0, 9, 1, 8, 8, 4, 256, 1, 0, null, 0, null) == _lib.ERR_BAD_ARG


def test_python_layer_refuses_cpu_tensors():
    import torch
    import vq_gemm_b200 as V
    x = torch.zeros(1, 8, dtype=torch.float16)
    idx = torch.zeros(4, 2, dtype=torch.uint8)
    cb = torch.zeros(1, 256, 4, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        V.vq_gemm(x, idx, cb)
    with pytest.raises(RuntimeError, match="no CPU path"):
        V.gemm(x, x.t().contiguous())


def test_routing_of_the_benchmark_configurations(lib):
    P = _lib.PATHS
    auto = lambda *a: lib.vqg_auto_path(*a)
    assert auto(16, 4096, 4096, 4, 256, 1, 0, 0) == P["decode"]          # C1: small matrix, 16 rows
    assert auto(1, 11008, 4096, 4, 256, 1, 128, 0) == P["decode"]        # C2
    assert auto(16, 8192, 8192, 8, 4096, 2, 0, 0) == P["small_ts"]       # C3: 4096-entry codebook
    assert auto(4096, 14336, 4096, 4, 256, 1, 128, 0) == P["tensor_ts"]  # C4
    assert auto(2048, 28672, 8192, 8, 256, 1, 128, 0) == P["tensor_ts"]  # C5
    assert auto(16, 28672, 8192, 8, 256, 1, 128, 0) == P["small_ts"]     # 16 rows on a large matrix
    assert auto(4, 28672, 8192, 8, 256, 1, 128, 0) == P["decode"]
    assert auto(8, 28672, 8192, 8, 256, 1, 128, 0) == P["decode"]        # up to 8 rows the decode kernel wins everywhere
    assert auto(16, 14336, 4096, 4, 256, 1, 128, 0) == P["decode"]       # 16 rows, one K chunk, replicated codebook
    assert auto(64, 28672, 8192, 8, 256, 1, 128, 0) == P["small_ts"]
    assert auto(128, 28672, 8192, 8, 256, 1, 128, 0) == P["tensor_ts"]
    assert auto(130, 96, 192, 4, 256, 1, 32, 0) == P["two_phase"]        # ragged K: dequantise, then the dense kernel
    assert auto(130, 96, 192, 3, 256, 1, 32, 0) == P["generic"]          # odd sub-vector length: CUDA-core kernel
    PK = _lib.IDX_PACKED12
    assert auto(16, 8192, 8192, 8, 4096, PK, 0, 0) == P["small_ts"]      # C3 with its indices packed
    assert auto(2048, 8192, 8192, 8, 4096, PK, 0, 0) == P["two_phase"]
    assert auto(16, 8192, 8192, 4, 4096, PK, 0, 0) == P["two_phase"]     # v = 4 has no packed tensor-memory instance
    assert auto(3, 100, 48, 4, 4096, PK, 0, 0) == P["generic"]
    assert auto(2048, 1280, 4096, 2, 256, 1, 0, 1) == P["two_phase"]     # the reference's own format
