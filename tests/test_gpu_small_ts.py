"""The small-batch kernel (M <= 128): weights through tensor memory, K loop split evenly over the SMs,
partial sums combined in contributor order.  Against the oracle, through the C ABI."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits, run_bl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N,v,C,rpc,dt", [
    (1, 128, 128, 4, 256, 128, torch.uint8),          # one tile, one stage, one CTA
    (1, 4096, 128, 4, 256, 128, torch.uint8),         # one tile split over 32 CTAs
    (3, 1024, 1280, 4, 256, 128, torch.uint8),        # 10 tiles x 8 stages over 80 CTAs
    (16, 4096, 4096, 4, 256, 0, torch.uint8),         # C1 shape: CTAs span tile boundaries
    (16, 2048, 512, 8, 4096, 0, torch.int16),         # unreplicated 64 KiB image, uint16 indices
    (7, 8192, 384, 8, 256, 128, torch.uint8),         # v = 8, uint8
    (16, 1024, 256, 8, 300, 128, torch.int16),        # small codebook behind uint16 indices (replicated)
    (17, 512, 256, 4, 256, 128, torch.uint8),         # 32 batch columns
    (64, 1024, 512, 8, 256, 256, torch.uint8),        # 64 batch columns, 256 rows per codebook
    (128, 2048, 1024, 4, 256, 128, torch.uint8),      # 128 batch columns
    (100, 256, 19072, 4, 100, 128, torch.uint8),      # more tiles than SMs, ragged batch, C not a power of two
    (16, 9728, 8192, 8, 256, 128, torch.uint8),       # large matrix: 256-wide pipeline stages (38 per tile, 64 tiles)
    (40, 5120, 15360, 4, 256, 128, torch.uint8),      # the same with v = 4 and 64 batch columns
])
def test_small_batch_matches_oracle(M, K, N, v, C, rpc, dt):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=M * 7 + N, idx_dtype=dt, cb_sigma=0.05)
    y = run_bl(V, x, idx, cb, rpc, path="small_ts")
    assert_within_tolerance(y, O.vq_gemm_bl(x, idx, cb, rpc))


def test_small_batch_deterministic_across_calls():
    x, idx, cb = O.make_bl_inputs(16, 8192, 1024, 8, 4096, 0, seed=3, idx_dtype=torch.int16)
    xs, ids, cbs = x.cuda(), idx.cuda(), cb.cuda()
    outs = [V.vq_gemm(xs, ids, cbs, layout="bl", path="small_ts").cpu() for _ in range(5)]
    for o in outs[1:]:
        assert torch.equal(bits(outs[0]), bits(o))
    assert V.device_status() == 0


def test_auto_route_for_batches_between_5_and_128():
    x, idx, cb = O.make_bl_inputs(48, 1024, 512, 4, 256, 128, seed=9)
    a = run_bl(V, x, idx, cb, 128, path="auto")
    b = run_bl(V, x, idx, cb, 128, path="small_ts")
    assert torch.equal(bits(a), bits(b))
    assert_within_tolerance(a, O.vq_gemm_bl(x, idx, cb, 128))


def test_rejects_shapes_outside_its_rules():
    x, idx, cb = O.make_bl_inputs(8, 192, 128, 4, 256, 128, seed=1)      # K not a multiple of 128
    with pytest.raises(RuntimeError, match="unsupported"):
        V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), layout="bl", path="small_ts")
    x, idx, cb = O.make_bl_inputs(200, 256, 128, 4, 256, 128, seed=1)    # M > 128
    with pytest.raises(RuntimeError, match="unsupported"):
        V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), layout="bl", path="small_ts")
