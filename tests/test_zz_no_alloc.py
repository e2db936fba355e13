"""The allocation-free small-batch entry point, called through the C ABI.

Some hosts cannot let a plugin call cudaMalloc: they reserve all of the GPU's memory for their
own pool at start-up, or they run the product on a path where the device-wide synchronisation of
cudaMalloc / cudaFree is not acceptable.  For them the library keeps the split-K scratch in a
fixed array of its own.  This test checks that entry point against the regular one (which takes a
caller-allocated workspace) on two consecutive calls -- the second call finds the array full of
the first call's partial sums and counters -- and that an oversized problem is refused.

The file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import pytest
import torch

from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits
from vq_gemm_b200 import _lib

pytestmark = pytest.mark.gpu


def _regular(lib, x, idx, cb, M, N, K, v, C, ib, rpc):
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    need = lib.vqg_workspace_bytes(M, N, K, v, C, ib, rpc, _lib.LAYOUT_BL, _lib.PATH_DECODE)
    ws = torch.zeros(max(need, 1), dtype=torch.uint8, device="cuda")
    st = lib.vqg_gemm_path(x.data_ptr(), idx.data_ptr(), cb.data_ptr(), y.data_ptr(), M, N, K, v, C, ib, rpc,
                           _lib.LAYOUT_BL, _lib.PATH_DECODE, ws.data_ptr(), ws.numel(),
                           torch.cuda.current_stream().cuda_stream)
    assert st == _lib.OK, _lib.status_string(st)
    torch.cuda.synchronize()
    return y


def _noalloc(lib, x, idx, cb, M, N, K, v, C, ib, rpc):
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    st = lib.vqg_gemm_small_batch_noalloc(x.data_ptr(), idx.data_ptr(), cb.data_ptr(), y.data_ptr(), M, N, K, v, C, ib,
                                          rpc, torch.cuda.current_stream().cuda_stream)
    assert st == _lib.OK, _lib.status_string(st)
    torch.cuda.synchronize()
    return y


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    lib = _lib.load()
    # first call: split-K over two chunks, uint16 indices into a 4096-entry codebook
    M, K, N, v, C, rpc = 16, 8192, 512, 8, 4096, 0
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=21, idx_dtype=torch.int16, cb_sigma=0.05)
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    a = _noalloc(lib, xd, idd, cbd, M, N, K, v, C, 2, rpc)
    b = _regular(lib, xd, idd, cbd, M, N, K, v, C, 2, rpc)
    assert torch.equal(bits(a), bits(b))          # same kernel, same summation order
    assert_within_tolerance(a.cpu(), O.vq_gemm_bl(x, idx, cb, rpc))

    # second call straight after: different shape, three chunks, scratch still holds the first call's data
    M2, K2, N2, v2, C2, rpc2 = 5, 4096 * 2 + 512, 256, 4, 256, 128
    x2, idx2, cb2 = O.make_bl_inputs(M2, K2, N2, v2, C2, rpc2, seed=22, cb_sigma=0.05)
    x2d, id2d, cb2d = x2.cuda(), idx2.cuda(), cb2.cuda()
    a2 = _noalloc(lib, x2d, id2d, cb2d, M2, N2, K2, v2, C2, 1, rpc2)
    b2 = _regular(lib, x2d, id2d, cb2d, M2, N2, K2, v2, C2, 1, rpc2)
    assert torch.equal(bits(a2), bits(b2))
    assert_within_tolerance(a2.cpu(), O.vq_gemm_bl(x2, idx2, cb2, rpc2))

    # and the first problem again: identical bits to its first run
    a3 = _noalloc(lib, xd, idd, cbd, M, N, K, v, C, 2, rpc)
    assert torch.equal(bits(a3), bits(a))


def test_noalloc_entry_without_split_k_and_limits():
    lib = _lib.load()
    M, K, N, v, C, rpc = 1, 4096, 1024, 4, 256, 128
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=23)
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    a = _noalloc(lib, xd, idd, cbd, M, N, K, v, C, 1, rpc)
    b = _regular(lib, xd, idd, cbd, M, N, K, v, C, 1, rpc)
    assert torch.equal(bits(a), bits(b))
    s = torch.cuda.current_stream().cuda_stream
    p = ctypes.c_void_p(xd.data_ptr())
    # few rows and a very long K: the chunks of K are handed over through scratch, 8 chunks x 16 x 12288 outputs
    # x 4 bytes = 6 MiB > 4 MiB: refused, nothing launched.  (Real buffers of the right size, so that a refusal
    # that failed to happen would still be a well-formed call.)
    Mb, Nb, Kb = 16, 12288, 32768
    need = lib.vqg_workspace_bytes(Mb, Nb, Kb, 8, 256, 1, 128, _lib.LAYOUT_BL, _lib.PATH_DECODE)
    assert need > (4 << 20)
    xb = torch.zeros((Mb, Kb), dtype=torch.float16, device="cuda")
    ib_ = torch.zeros((Nb, Kb // 8), dtype=torch.uint8, device="cuda")
    cbb = torch.zeros((Nb // 128, 256, 8), dtype=torch.float16, device="cuda")
    yb = torch.zeros((Mb, Nb), dtype=torch.float16, device="cuda")
    before = lib.vqg_launch_count()
    st = lib.vqg_gemm_small_batch_noalloc(xb.data_ptr(), ib_.data_ptr(), cbb.data_ptr(), yb.data_ptr(), Mb, Nb, Kb, 8, 256, 1,
                                          128, s)
    assert st == _lib.ERR_TOO_LARGE and "static buffer" in _lib.status_string(st)
    assert lib.vqg_launch_count() == before
    del xb, ib_, cbb, yb
    # shapes outside the small-batch kernel are refused too (no other kernel behind this entry)
    assert lib.vqg_gemm_small_batch_noalloc(p, p, p, p, 17, 1024, 4096, 4, 256, 1, 128, s) == _lib.ERR_UNSUPPORTED
    assert lib.vqg_gemm_small_batch_noalloc(p, p, p, p, 4, 1024, 4096 + 64, 4, 256, 1, 128, s) == _lib.ERR_UNSUPPORTED


def test_noalloc_calls_leave_free_device_memory_unchanged():
    """After the first call on the device (which is when the runtime loads the library's module and its fixed
    array), further calls must not change the amount of free device memory: a host that has given the rest of
    the GPU to its own pool can keep calling."""
    lib = _lib.load()
    M, K, N, v, C, rpc = 4, 8192, 512, 4, 256, 128          # split-K through the fixed array
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=31)
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream

    def call():
        st = lib.vqg_gemm_small_batch_noalloc(xd.data_ptr(), idd.data_ptr(), cbd.data_ptr(), y.data_ptr(), M, N, K, v, C, 1,
                                              rpc, s)
        assert st == _lib.OK, _lib.status_string(st)
        torch.cuda.synchronize()

    call()                                                   # first call: module load, address lookup
    free0 = torch.cuda.mem_get_info()[0]
    call()
    free1 = torch.cuda.mem_get_info()[0]
    call()
    free2 = torch.cuda.mem_get_info()[0]
    assert free0 == free1 == free2
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, rpc))
    assert "memory" in _lib.status_string(8)                 # VQG_ERR_NO_MEMORY has its own message
