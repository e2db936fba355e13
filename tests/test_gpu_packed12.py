"""12-bit indices packed two to three bytes, consumed by the product and dequantisation kernels directly: results
must equal what the same indices give when held in uint16 (dequantised weights bit for bit, products bit for bit
where the same kernel runs, within the tolerance otherwise), with the packing done by the CPU restatement."""
import numpy as np
import pytest
import torch

import vq_gemm_b200 as V
from oracle import quantize_oracle as Q
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits

pytestmark = pytest.mark.gpu


def _packed(idx):
    return torch.from_numpy(Q.pack12(idx.numpy()))


@pytest.mark.parametrize("N,K,v,C,rpc", [
    (256, 512, 8, 4096, 0),
    (384, 1024, 8, 1000, 128),      # groups, C not a power of two
    (100, 48, 4, 4096, 0),
    (33, 40, 2, 300, 11),
    (2048, 2048, 8, 4096, 0),
])
def test_dequant_of_packed_indices_is_bit_exact(N, K, v, C, rpc):
    _, idx, cb = O.make_bl_inputs(1, K, N, v, C, rpc, seed=N + K, idx_dtype=torch.int16)
    w = V.dequant(_packed(idx).cuda(), cb.cuda(), rows_per_codebook=rpc, index_bits=12)
    assert torch.equal(bits(w), bits(O.dequant_bl_layout(idx, cb, rpc)))


@pytest.mark.parametrize("M,N,K,v,C,rpc,path", [
    (16, 1024, 1024, 8, 4096, 0, "small_ts"),
    (1, 512, 2048, 8, 4096, 0, "small_ts"),
    (100, 256, 512, 8, 1000, 128, "small_ts"),
    (128, 384, 256, 8, 256, 128, "small_ts"),      # a small codebook in packed form still takes the unreplicated image
    (16, 256, 384, 8, 4096, 0, "small_ts"),        # rows of 72 bytes: neighbouring rows sit differently in their 16-byte chunks
    (3, 128, 128, 8, 512, 0, "small_ts"),          # one pipeline stage per row
    (40, 640, 896, 8, 4096, 128, "small_ts"),
    (300, 512, 1024, 8, 4096, 0, "two_phase"),
    (64, 256, 256, 4, 2048, 0, "two_phase"),       # v = 4: no tensor-memory instance, dequantise first
    (5, 96, 40, 4, 3000, 0, "generic"),
    (7, 33, 24, 2, 4096, 11, "generic"),
])
def test_product_with_packed_indices(M, N, K, v, C, rpc, path):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=M + N, idx_dtype=torch.int16)
    pk = _packed(idx).cuda()
    assert V.auto_path(M, N, K, v, C, 12, rpc) == path
    y = V.vq_gemm(x.cuda(), pk, cb.cuda(), rows_per_codebook=rpc, index_bits=12)
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, rpc))
    # the same route on uint16 storage gives the same bits (same kernel, same order of operations)
    y16 = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=rpc, path=path)
    assert torch.equal(bits(y), bits(y16))
    assert V.device_status() == 0


def test_c3_shape_packed_whole_output():
    x, idx, cb = O.make_bl_inputs(16, 8192, 8192, 8, 4096, 0, seed=0, idx_dtype=torch.int16)
    pk = V.quantize.pack12(idx.cuda())
    assert pk.shape == (8192, 1536) and np.array_equal(pk[:4].cpu().numpy(), Q.pack12(idx[:4].numpy()))
    y = V.vq_gemm(x.cuda(), pk, cb.cuda(), index_bits=12)
    y16 = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), path="small_ts")
    assert torch.equal(bits(y), bits(y16))
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, 0))


def test_golden_fixture():
    from tests._util import load_golden
    g = load_golden("bl_v8_c4096_packed12")
    w = V.dequant(g["packed"].cuda(), g["codebook"].cuda(), rows_per_codebook=0, index_bits=12)
    assert torch.equal(bits(w), bits(g["w_decoded"]))
    y = V.vq_gemm(g["x"].cuda(), g["packed"].cuda(), g["codebook"].cuda(), index_bits=12)
    assert_within_tolerance(y.cpu(), g["y"])


def test_argument_checks():
    x, idx, cb = O.make_bl_inputs(4, 64, 32, 8, 4096, 0, seed=1, idx_dtype=torch.int16)
    pk = _packed(idx).cuda()
    with pytest.raises(RuntimeError):
        V.vq_gemm(x.cuda(), pk, cb.cuda(), index_bits=10)
    with pytest.raises(RuntimeError):
        V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), index_bits=12)          # not a packed tensor
    with pytest.raises(RuntimeError):
        V.vq_gemm(x.cuda(), pk, cb.cuda(), index_bits=12, layout="ref")
    # a 12-bit value above the codebook's size (malformed input) reads entry 0, never past the image
    small = cb[:, :100].contiguous()
    w = V.dequant(pk, small.cuda(), index_bits=12)
    ref = O.dequant_bl_layout(torch.where(idx >= 100, torch.zeros_like(idx), idx), small, 0)
    assert torch.equal(bits(w), bits(ref))
