"""The M <= 16 kernel (index streaming + codebook lookups + mma.sync, split-K) against the oracle."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits, run_bl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N,v,C,rpc,dt", [
    (1, 256, 16, 4, 256, 0, torch.uint8),           # one slice, one row block
    (1, 1024, 256, 4, 256, 128, torch.uint8),       # 4 slices -> 4 row blocks side by side
    (3, 4096, 512, 4, 256, 128, torch.uint8),       # full 16-slice chunk
    (8, 2048, 384, 8, 256, 128, torch.uint8),       # v = 8, uint8
    (16, 4096, 256, 4, 256, 0, torch.uint8),        # two batch tiles
    (9, 512, 48, 4, 256, 16, torch.uint8),          # group of 16 rows
    (16, 2048, 128, 8, 4096, 0, torch.int16),       # large codebook, uint16
    (5, 8192, 256, 8, 4096, 0, torch.int16),        # split-K (2 chunks)
    (16, 8192, 64, 4, 256, 0, torch.uint8),         # split-K, v = 4
    (2, 4096 + 256, 32, 4, 256, 0, torch.uint8),    # second chunk holds a single slice
    (4, 1024, 64, 4, 100, 0, torch.uint8),          # C not a power of two
    (1, 768, 80, 4, 256, 0, torch.uint8),           # 3 slices: warps left idle
    (7, 1024, 64, 8, 300, 32, torch.int16),         # small codebook behind uint16 indices
    (4, 2048, 128, 4, 256, 128, torch.uint8),       # largest batch of the two-columns-per-row form
    (12, 1024, 96, 8, 256, 32, torch.uint8),        # batch rows above 8 with v = 8
    (3, 8192, 14336, 8, 256, 128, torch.uint8),     # many row blocks, 2 chunks: a CTA keeps its rows' sums across chunks
    (16, 12288, 14336, 4, 256, 128, torch.uint8),   # the same with 3 chunks, 16 batch rows, v = 4
    (8, 8192, 14336, 8, 4096, 0, torch.int16),      # the same with a single large codebook
    (2, 8192 + 512, 14464, 4, 256, 128, torch.uint8),  # the same with a short last chunk and row blocks not a multiple of the SM count
])
def test_decode_matches_oracle(M, K, N, v, C, rpc, dt):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=M * 131 + N, idx_dtype=dt, cb_sigma=0.05)
    y = run_bl(V, x, idx, cb, rpc, path="decode")
    assert_within_tolerance(y, O.vq_gemm_bl(x, idx, cb, rpc))


def test_decode_is_what_auto_picks_for_small_m():
    x, idx, cb = O.make_bl_inputs(2, 1024, 128, 4, 256, 128, seed=1)
    a = run_bl(V, x, idx, cb, 128, path="auto")
    d = run_bl(V, x, idx, cb, 128, path="decode")
    assert torch.equal(bits(a), bits(d))


def test_uint16_indices_with_v4_go_to_the_generic_kernel():
    x, idx, cb = O.make_bl_inputs(3, 512, 64, 4, 300, 0, seed=2, idx_dtype=torch.int16, cb_sigma=0.05)
    with pytest.raises(RuntimeError, match="unsupported"):
        V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), layout="bl", path="decode")
    assert_within_tolerance(run_bl(V, x, idx, cb, 0, path="auto"), O.vq_gemm_bl(x, idx, cb, 0))


def test_decode_rejects_unsupported_shapes():
    x, idx, cb = O.make_bl_inputs(2, 128, 16, 4, 256, 0, seed=1)  # K not a multiple of 256
    with pytest.raises(RuntimeError, match="unsupported"):
        V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), layout="bl", path="decode")
    # auto falls through to the generic kernel for the same shape
    assert_within_tolerance(run_bl(V, x, idx, cb, 0, path="auto"), O.vq_gemm_bl(x, idx, cb, 0))


def test_decode_deterministic_including_split_k():
    # the reference's determinism check (bench.py:118-132): repeated calls give identical bits
    x, idx, cb = O.make_bl_inputs(16, 8192, 512, 8, 4096, 0, seed=4, idx_dtype=torch.int16)
    xs, ids, cbs = x.cuda(), idx.cuda(), cb.cuda()
    outs = [V.vq_gemm(xs, ids, cbs, layout="bl", path="decode").cpu() for _ in range(5)]
    for o in outs[1:]:
        assert torch.equal(bits(outs[0]), bits(o))
    assert V.device_status() == 0


def test_decode_linearity_in_x():
    # size-independent property: Y(2*X) == 2*Y(X) bit for bit (power-of-two scaling is exact in fp16/fp32)
    x, idx, cb = O.make_bl_inputs(4, 4096, 1024, 4, 256, 128, seed=6)
    y1 = run_bl(V, x, idx, cb, 128, path="decode")
    y2 = run_bl(V, (x.float() * 2).half(), idx, cb, 128, path="decode")
    normal = y1.abs() >= 2.0 ** -13   # fp16-subnormal outputs round on a fixed grid
    assert torch.equal((y1.float() * 2).half()[normal], y2[normal])
    assert float((y1.float() * 2 - y2.float()).abs().max()) <= 2.0 ** -23
