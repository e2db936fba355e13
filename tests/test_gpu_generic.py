"""The shape-agnostic kernel against the oracle: ragged and tiny shapes, both weight formats."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, load_golden, run_bl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tag", ["bl_v4_c256_groups", "bl_v8_c4096_single", "bl_v8_c256_groups"])
def test_bl_golden(tag):
    g = load_golden(tag)
    rpc = int(g["meta"][5])
    y = run_bl(V, g["x"], g["idx"], g["codebook"], rpc, path="generic")
    assert_within_tolerance(y, g["y"], tag)


@pytest.mark.parametrize("tag", ["ref_small", "ref_two_tiles", "ref_ragged"])
def test_ref_golden(tag):
    g = load_golden(tag)
    y = V.vq_gemm(g["x"].cuda(), g["w"].cuda(), g["codebook"].cuda(), layout="ref", path="generic").cpu()
    assert_within_tolerance(y, g["y"], tag)
    # e2e_gemm infers the reference format from the shapes
    y2 = V.e2e_gemm(g["x"].cuda(), g["w"].cuda(), g["codebook"].cuda()).cpu()
    assert_within_tolerance(y2, g["y"], tag)


@pytest.mark.parametrize("M,K,N,v,C,rpc,dt", [
    (1, 8, 1, 4, 256, 0, torch.uint8),
    (7, 36, 19, 4, 100, 0, torch.uint8),
    (65, 130, 67, 2, 256, 0, torch.uint8),
    (3, 64, 96, 8, 4096, 32, torch.int16),
])
def test_ragged(M, K, N, v, C, rpc, dt):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=M + N, idx_dtype=dt, cb_sigma=0.5)
    y = run_bl(V, x, idx, cb, rpc, path="generic")
    assert_within_tolerance(y, O.vq_gemm_bl(x, idx, cb, rpc))


def test_empty_and_zero_k():
    cb = torch.zeros(1, 256, 4, dtype=torch.float16).cuda()
    y = V.vq_gemm(torch.zeros(0, 16, dtype=torch.float16).cuda(), torch.zeros(8, 4, dtype=torch.uint8).cuda(), cb,
                  layout="bl")
    assert y.shape == (0, 8)
    y = V.vq_gemm(torch.zeros(4, 0, dtype=torch.float16).cuda(), torch.zeros(8, 0, dtype=torch.uint8).cuda(), cb,
                  layout="bl")
    assert y.shape == (4, 8) and float(y.abs().max()) == 0.0
