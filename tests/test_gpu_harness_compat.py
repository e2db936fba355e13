"""Drives the PyTorch-extension shim the way the reference's harness does (bench.py:62-139):
alias modules under the reference's six names, its default shape and seed, `e2e_gemm(input, w,
codebook)`, the 5-run determinism check and the plain `gemm` mode."""
import os
import sys

import pytest
import torch

from oracle import vq_oracle as O
from tests._util import ROOT, assert_within_tolerance, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def modules():
    if not os.path.exists(os.path.join(ROOT, "vq_gemm_cuda.so")):
        pytest.fail("vq_gemm_cuda.so is missing: run `python compile_kernels.py build_ext --inplace`")
    sys.path.insert(0, os.path.join(ROOT, "compat"))
    try:
        import vq_gemm_cuda_cublas_gemm, vq_gemm_cuda_s1, vq_gemm_cuda_s2_128, vq_gemm_cuda_s2_512  # noqa: E401
        import vq_gemm_cuda_s3_naive, vq_gemm_cuda_s3_wasp  # noqa: E401
    finally:
        sys.path.pop(0)
    return {"cublas": vq_gemm_cuda_cublas_gemm, "s1": vq_gemm_cuda_s1, "s2_128": vq_gemm_cuda_s2_128,
            "s2_512": vq_gemm_cuda_s2_512, "s3_naive": vq_gemm_cuda_s3_naive, "s3_wasp": vq_gemm_cuda_s3_wasp}


def test_default_shape_like_the_reference_harness(modules):
    M, K, N, ENTRY, RATIO = 2048, 4096, 640, 256, 2          # bench.py:13-15,29-30
    torch.manual_seed(42)                                     # bench.py:33
    dev = torch.device("cuda")
    inp = torch.randn(M, K, dtype=torch.float16, device=dev)  # bench.py:83-85
    w = torch.randint(0, ENTRY, (K, N), dtype=torch.uint8, device=dev)
    codebook = torch.randn(N // 4, ENTRY, RATIO, dtype=torch.float16, device=dev)
    out = modules["s3_wasp"].e2e_gemm(inp, w, codebook)
    torch.cuda.synchronize()
    assert out.shape == (M, N * RATIO) and out.dtype == torch.float16
    ref = O.vq_gemm_ref_layout(inp.cpu(), w.cpu(), codebook.cpu())
    assert_within_tolerance(out.cpu(), ref)
    outs = [modules["s1"].e2e_gemm(inp, w, codebook).cpu() for _ in range(5)]  # bench.py:118-127
    for o in outs[1:]:
        assert torch.equal(bits(outs[0]), bits(o))


def test_plain_gemm_mode(modules):
    M = N = K = 1024                                          # bench.py:18-19 uses 4096; smaller here
    torch.manual_seed(42)
    inp = torch.randn(M, K, dtype=torch.float16, device="cuda")
    w = torch.rand(K, N, dtype=torch.float16, device="cuda")  # bench.py:137
    out = modules["s1"].gemm(inp, w)
    ref = modules["cublas"].gemm(inp, w)
    assert torch.equal(bits(out), bits(ref))
    assert_within_tolerance(out.cpu(), (inp.cpu().float() @ w.cpu().float()).half())


def test_generalised_entry_point_and_errors(modules):
    x, idx, cb = O.make_bl_inputs(4, 1024, 256, 4, 256, 128, seed=0)
    y = modules["s2_128"].vq_gemm(x.cuda(), idx.cuda(), cb.cuda())
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, 128))
    wd = modules["s2_128"].dequant(idx.cuda(), cb.cuda())
    assert torch.equal(bits(wd), bits(O.dequant_bl_layout(idx, cb, 128)))
    with pytest.raises(RuntimeError):
        modules["s1"].e2e_gemm(x, idx, cb)  # CPU tensors
    with pytest.raises(RuntimeError):
        modules["s1"].e2e_gemm(x.cuda(), idx.cuda()[:, :7].contiguous(), cb.cuda())  # shapes fit neither format
