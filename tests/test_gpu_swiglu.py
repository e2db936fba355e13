"""Gated product SiLU(X g) * (X u): fused epilogue of the prefill kernel and the two-kernel route."""
import ctypes

import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits
from vq_gemm_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(x, idx, cb, rpc):
    y = V.vq_gemm_swiglu(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=rpc)
    torch.cuda.synchronize()
    assert V.device_status() == 0
    return y.cpu()


@pytest.mark.parametrize("M,K,N,v,rpc", [
    (300, 1024, 1280, 8, 128),     # fused: 10 tiles over 20 CTA pairs, every tile summed from two partials
    (700, 2048, 1024, 4, 128),     # fused: uneven split, tiles shared by several pairs
    (2048, 512, 4608, 8, 128),     # fused: whole tiles and shared tiles mixed, 18 x 8 tiles
    (256, 512, 512, 4, 0),         # fused, single codebook
    (8, 1024, 512, 4, 128),        # decode kernel + elementwise kernel
    (64, 1024, 512, 8, 128),       # small-batch tensor-memory kernel + elementwise kernel
    (130, 192, 96, 4, 32),         # generic kernel + elementwise kernel
])
def test_gated_product_matches_oracle(M, K, N, v, rpc):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, rpc, seed=M + N, cb_sigma=0.05)
    ref = O.vq_gemm_swiglu_bl(x, idx, cb, rpc)
    y = _run(x, idx, cb, rpc)
    assert y.shape == (M, N // 2)
    assert_within_tolerance(y, ref)
    assert torch.equal(bits(_run(x, idx, cb, rpc)), bits(y))


def test_fused_epilogue_equals_product_then_elementwise():
    # same accumulators; the fused route skips the fp16 rounding of the two products
    M, K, N, v, rpc = 512, 1024, 1024, 8, 128
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, rpc, seed=5, cb_sigma=0.05)
    fused = _run(x, idx, cb, rpc)
    p = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=rpc, layout="bl").float()
    two_step = (torch.nn.functional.silu(p[:, 0::2]) * p[:, 1::2]).half().cpu()
    assert float((fused.float() - two_step.float()).abs().max()) <= 4e-3 * float(two_step.float().abs().max()) + 1e-3


def test_whole_tile_schedule_without_workspace_partials():
    # a workspace too small for the partial tiles makes the kernel keep whole tiles: same result within rounding
    M, K, N, v, rpc = 300, 1024, 1280, 8, 128
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, rpc, seed=6, cb_sigma=0.05)
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    y = torch.empty(M, N // 2, dtype=torch.float16, device="cuda")
    st = _lib.load().vqg_gemm_swiglu(xd.data_ptr(), idd.data_ptr(), cbd.data_ptr(), y.data_ptr(), M, N // 2, K, v, 256, 1, rpc,
                                     None, 0, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert_within_tolerance(y.cpu(), O.vq_gemm_swiglu_bl(x, idx, cb, rpc))


def test_interleave_and_argument_checks():
    g = torch.arange(6).reshape(3, 2)
    u = g + 100
    assert V.interleave_gate_up(g, u).tolist() == [[0, 1], [100, 101], [2, 3], [102, 103], [4, 5], [104, 105]]
    x, idx, cb = O.make_bl_inputs(4, 64, 6, 4, 256, 0, seed=1)
    with pytest.raises(RuntimeError):
        V.vq_gemm_swiglu(x.cuda(), idx[:5].contiguous().cuda(), cb.cuda())        # odd number of weight rows
    lib = _lib.load()
    p = ctypes.c_void_p(4096)
    assert lib.vqg_gemm_swiglu(p, p, p, p, 4, -1, 64, 4, 256, 1, 0, None, 0, None) == _lib.ERR_BAD_ARG
    assert lib.vqg_gemm_swiglu(p, p, p, p, 4, 0, 64, 4, 256, 1, 0, None, 0, None) == _lib.OK
