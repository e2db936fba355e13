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


@pytest.mark.parametrize("K,Nq", [(64, 64), (100, 12), (4096, 640)])
def test_ref_random(K, Nq):
    _, w, cb = O.make_ref_inputs(1, K, Nq, seed=K + Nq)
    out = V.dequant(w.cuda(), cb.cuda(), layout="ref")
    assert torch.equal(bits(out), bits(O.dequant_ref_layout(w, cb)))


def test_empty():
    idx = torch.zeros(0, 16, dtype=torch.uint8).cuda()
    cb = torch.zeros(1, 256, 4, dtype=torch.float16).cuda()
    assert V.dequant(idx, cb).shape == (0, 64)
