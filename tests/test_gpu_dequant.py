"""Dequantised weights must match the oracle bit for bit (pure gather), through the C ABI."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import bits, load_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tag", ["bl_v4_c256_groups", "bl_v8_c4096_single", "bl_v8_c256_groups"])
def test_bl_golden(tag):
    g = load_golden(tag)
    rpc = int(g["meta"][5])
    w = V.dequant(g["idx"].cuda(), g["codebook"].cuda(), rows_per_codebook=rpc)
    assert torch.equal(bits(w), bits(g["w_decoded"]))


def test_bl_dequant_matches_bytes_gathered_by_the_reference():
    # Nq = 4: the reference's gather (bench.py:46-55) with its single codebook IS the generalised rule with v = 2
    g = load_golden("ref_nq4_bridge")
    w = V.dequant(g["w"].cuda(), g["codebook"][0].contiguous().cuda(), rows_per_codebook=0, layout="bl")
    assert torch.equal(bits(w), bits(g["w_decoded"]))
    # and a product through that gather: Y = X8 @ W^T with W = the reference's bytes
    x8 = g["x"][:, :8].contiguous()
    y = V.vq_gemm(x8.cuda(), g["w"].cuda(), g["codebook"][0].contiguous().cuda(), rows_per_codebook=0, layout="bl")
    assert O.check_tolerance(y.cpu(), O.matmul_fp32acc(x8, g["w_decoded"]))["ok"]


@pytest.mark.parametrize("tag", ["ref_small", "ref_two_tiles", "ref_ragged", "ref_nq4_bridge"])
def test_ref_golden_from_reference_gather(tag):
    g = load_golden(tag)
    w = V.dequant(g["w"].cuda(), g["codebook"].cuda(), layout="ref")
    assert torch.equal(bits(w), bits(g["w_decoded"]))


@pytest.mark.parametrize("N,K,v,C,rpc,dt", [
    (256, 512, 4, 256, 128, torch.uint8),
    (384, 256, 8, 256, 128, torch.uint8),
    (128, 1024, 8, 4096, 0, torch.int16),
    (100, 40, 4, 200, 0, torch.uint8),        # ragged N, small C
    (33, 24, 2, 256, 11, torch.uint8),        # v = 2, odd group size
    (64, 64, 4, 1000, 16, torch.int16),       # uint16 indices, C not a power of two
    (48, 16, 8, 60000, 0, torch.int16),       # codebook too large for shared memory; indices above 32767
    (2048, 4096, 4, 256, 128, torch.uint8),
])
def test_bl_random(N, K, v, C, rpc, dt):
    _, idx, cb = O.make_bl_inputs(1, K, N, v, C, rpc, seed=N * 3 + K, idx_dtype=dt)
    w = V.dequant(idx.cuda(), cb.cuda(), rows_per_codebook=rpc)
    assert torch.equal(bits(w), bits(O.dequant_bl_layout(idx, cb, rpc)))


@pytest.mark.parametrize("K,Nq", [(64, 64), (100, 12), (4096, 640), (72, 132), (8192, 8), (130, 260), (1, 4), (200, 1028)])
def test_ref_random(K, Nq):
    _, w, cb = O.make_ref_inputs(1, K, Nq, seed=K + Nq)
    out = V.dequant(w.cuda(), cb.cuda(), layout="ref")
    assert torch.equal(bits(out), bits(O.dequant_ref_layout(w, cb)))


def test_ref_misaligned_pointers_take_the_plain_kernel():
    # index matrix starting on an odd byte: the streaming form (4-byte index words) must not be chosen
    _, w, cb = O.make_ref_inputs(1, 96, 136, seed=5)
    buf = torch.empty(w.numel() + 1, dtype=torch.uint8, device="cuda")
    wd = buf[1:].view(96, 136)
    wd.copy_(w)
    assert wd.data_ptr() % 4 != 0
    out = V.dequant(wd, cb.cuda(), layout="ref")
    assert torch.equal(bits(out), bits(O.dequant_ref_layout(w, cb)))


@pytest.mark.parametrize("K,Nq", [(64, 16), (256, 144), (512, 640), (192, 272), (4096, 128)])
def test_ref_transposed_weights_through_an_identity_product(K, Nq):
    # the K-major form of the dequantised reference weights only exists as the operand of the dense kernel:
    # with X = I the product returns it element for element (one non-zero term per sum, exact in fp32)
    _, w, cb = O.make_ref_inputs(1, K, Nq, seed=3 * K + Nq)
    x = torch.eye(K, dtype=torch.float16)
    y = V.vq_gemm(x.cuda(), w.cuda(), cb.cuda(), layout="ref")
    assert torch.equal(y.cpu(), O.dequant_ref_layout(w, cb))


@pytest.mark.parametrize("N,K,v,C,rpc,dt,S", [
    (512, 1024, 8, 4096, 0, torch.int16, 1),      # streaming form, one 64 KiB image
    (300, 512, 8, 1024, 100, torch.int16, 1),     # groups of 100 rows: block ranges cross group boundaries
    (1000, 256, 4, 512, 0, torch.int16, 1),
    (777, 64, 2, 2048, 77, torch.int16, 1),
    (2048, 2048, 8, 256, 128, torch.uint8, 2),    # residual, replicated images
    (640, 512, 4, 256, 128, torch.uint8, 3),
    (200, 128, 2, 256, 0, torch.uint8, 2),
    (256, 512, 8, 4096, 0, torch.int16, 2),       # residual with large codebooks: unreplicated images
    (96, 256, 8, 8192, 0, torch.int16, 2),        # images do not fit: plain kernel
    (64, 24, 8, 256, 0, torch.uint8, 2),
    (512, 256, 4, 256, 128, torch.uint8, 4),
    (256, 128, 8, 256, 64, torch.uint8, 5),       # more than four stages: plain kernel
    (130, 64, 2, 300, 0, torch.int16, 8),
])
def test_bl_streaming_form(N, K, v, C, rpc, dt, S):
    if S == 1:
        _, idx, cb = O.make_bl_inputs(1, K, N, v, C, rpc, seed=N + K, idx_dtype=dt)
        w = V.dequant(idx.cuda(), cb.cuda(), rows_per_codebook=rpc)
        assert torch.equal(bits(w), bits(O.dequant_bl_layout(idx, cb, rpc)))
    else:
        _, idx, cb = O.make_residual_inputs(1, K, N, v, C, rpc, S, seed=N + K, idx_dtype=dt)
        w = V.dequant_residual(idx.cuda(), cb.cuda(), rows_per_codebook=rpc)
        assert torch.equal(bits(w), bits(O.dequant_bl_residual(idx, cb, rpc)))


@pytest.mark.parametrize("C,dt", [(100, torch.uint8), (1000, torch.int16)])
def test_indices_beyond_the_codebook_read_its_last_entry(C, dt):
    # malformed input: the streaming kernel keeps its lookups inside the shared-memory image
    _, idx, cb = O.make_bl_inputs(1, 256, 128, 8, C, 0, seed=C, idx_dtype=dt)
    bad = idx.clone()
    bad[3, 5] = C + 7 if dt == torch.uint8 else 30000
    bad[100, 0] = C
    w = V.dequant(bad.cuda(), cb.cuda(), rows_per_codebook=0)
    fixed = idx.clone()
    fixed[3, 5] = C - 1
    fixed[100, 0] = C - 1
    assert torch.equal(bits(w), bits(O.dequant_bl_layout(fixed, cb, 0)))


def test_indices_beyond_the_codebook_in_the_plain_kernels():
    # K/v = 7 is not a whole number of 16-byte outputs: the plain dequant kernel; and the shape-agnostic product
    x, idx, cb = O.make_bl_inputs(3, 14, 40, 2, 50, 0, seed=4)
    bad, fixed = idx.clone(), idx.clone()
    bad[7, 3], fixed[7, 3] = 250, 49
    w = V.dequant(bad.cuda(), cb.cuda(), rows_per_codebook=0)
    assert torch.equal(bits(w), bits(O.dequant_bl_layout(fixed, cb, 0)))
    y = V.vq_gemm(x.cuda(), bad.cuda(), cb.cuda(), rows_per_codebook=0, path="generic")
    assert O.check_tolerance(y.cpu(), O.vq_gemm_bl(x, fixed, cb, 0))["ok"]


def test_empty():
    idx = torch.zeros(0, 16, dtype=torch.uint8).cuda()
    cb = torch.zeros(1, 256, 4, dtype=torch.float16).cuda()
    assert V.dequant(idx, cb).shape == (0, 64)
