"""Indices that name entries beyond the codebook are the caller's error; the kernels must still complete (16-bit
and packed indices are clamped to the last entry, 8-bit ones address inside the block's shared memory) and every
output column that does not involve the bad index must be right."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,v,C,rpc,dt,path", [
    (1, 512, 1024, 4, 37, 128, torch.uint8, "decode"),        # small codebooks, two image slots
    (8, 256, 512, 8, 100, 0, torch.uint8, "decode"),
    (4, 256, 1024, 8, 1000, 0, torch.int16, "decode"),
    (16, 256, 512, 8, 1000, 0, torch.int16, "small_ts"),
    (64, 256, 256, 4, 100, 128, torch.uint8, "small_ts"),
    (256, 512, 512, 4, 100, 128, torch.uint8, "tensor_ts"),
    (256, 512, 512, 8, 60, 128, torch.uint8, "tensor_pair"),
    (130, 256, 256, 4, 100, 128, torch.uint8, "tensor"),
])
def test_launch_completes_and_other_columns_are_right(M, N, K, v, C, rpc, dt, path):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=M + N + C, idx_dtype=dt)
    bad = idx.clone()
    rows = [3, N // 2, N - 1]
    for r in rows:
        bad[r, 1] = 255 if dt == torch.uint8 else 30000
    y = V.vq_gemm(x.cuda(), bad.cuda(), cb.cuda(), rows_per_codebook=rpc, path=path)
    torch.cuda.synchronize()
    assert V.device_status() == 0
    ref = O.vq_gemm_bl(x, idx, cb, rpc)
    keep = torch.ones(N, dtype=torch.bool)
    keep[rows] = False
    assert_within_tolerance(y.cpu()[:, keep], ref[:, keep])
    if dt != torch.uint8:      # clamped: the bad index reads the last entry
        fixed = idx.clone()
        for r in rows:
            fixed[r, 1] = C - 1
        assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, fixed, cb, rpc))
    # the context is intact: the same call with the right indices
    y2 = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=rpc, path=path)
    assert_within_tolerance(y2.cpu(), ref)
