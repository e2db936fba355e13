"""Residual (multi-codebook) weights through the C ABI: dequantised weights bit for bit against the format's
rule, products against the oracle on every route -- decode kernel (stages walked like chunks of K), prefill
kernel (two resident codebook images, HADD2 before the tensor-memory store), dequantise + dense, generic."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits, load_golden

pytestmark = pytest.mark.gpu


def _run(x, idx, cb, rpc):
    y = V.vq_gemm_residual(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=rpc)
    torch.cuda.synchronize()
    assert V.device_status() == 0
    return y.cpu()


def test_golden_fixture_of_the_scalar_rule():
    g = load_golden("bl_residual_v8_c256_s2")
    M, K, N, v, C, rpc, stages, seed = [int(t) for t in g["meta"]]
    w = V.dequant_residual(g["idx"].cuda(), g["codebook"].cuda(), rows_per_codebook=rpc)
    assert torch.equal(bits(w), bits(g["w_decoded"]))
    assert_within_tolerance(_run(g["x"], g["idx"], g["codebook"], rpc), g["y"])


@pytest.mark.parametrize("N,K,v,C,rpc,S,dt", [
    (256, 512, 8, 256, 128, 2, torch.uint8),
    (384, 256, 4, 256, 128, 2, torch.uint8),
    (64, 1024, 8, 4096, 0, 2, torch.int16),
    (100, 40, 4, 200, 0, 3, torch.uint8),         # ragged, three stages
    (33, 24, 2, 256, 11, 2, torch.uint8),         # v = 2, odd group size
])
def test_dequantised_weights_are_bit_exact(N, K, v, C, rpc, S, dt):
    _, idx, cb = O.make_residual_inputs(1, K, N, v, C, rpc, stages=S, seed=N + K, idx_dtype=dt)
    w = V.dequant_residual(idx.cuda(), cb.cuda(), rows_per_codebook=rpc)
    assert torch.equal(bits(w), bits(O.dequant_bl_residual(idx, cb, rpc)))


@pytest.mark.parametrize("M,K,N,v,C,rpc,S,dt", [
    (1, 4096, 512, 4, 256, 128, 2, torch.uint8),       # decode, M <= 4 form, one K chunk per stage
    (3, 8192, 256, 8, 256, 128, 2, torch.uint8),       # decode, two K chunks x two stages through the workspace
    (16, 2048, 256, 8, 4096, 0, 2, torch.int16),       # decode, 16 rows, 4096-entry codebooks
    (8, 1024, 128, 4, 256, 0, 3, torch.uint8),         # decode, three stages, single codebook per stage
    (2, 8192, 14336, 8, 256, 128, 2, torch.uint8),     # decode, many row blocks: running sums on chip over 4 chunks
    (300, 1024, 768, 8, 256, 128, 2, torch.uint8),     # prefill kernel, v = 8
    (512, 512, 512, 4, 256, 128, 2, torch.uint8),      # prefill kernel, v = 4
    (2048, 2048, 1024, 8, 256, 128, 2, torch.uint8),   # prefill kernel, K loops dealt out over the pairs
    (64, 1024, 512, 8, 256, 128, 2, torch.uint8),      # prefill kernel below 128 batch rows
    (256, 512, 256, 8, 4096, 0, 2, torch.int16),       # 16-bit indices: dequantise, then the dense kernel
    (256, 512, 256, 8, 256, 128, 3, torch.uint8),      # three stages above 16 rows: dequantise, then dense
    (130, 96, 192, 4, 256, 32, 2, torch.uint8),        # ragged K: generic kernel
])
def test_product_matches_oracle(M, K, N, v, C, rpc, S, dt):
    x, idx, cb = O.make_residual_inputs(M, K, N, v, C, rpc, stages=S, seed=M * 3 + N, idx_dtype=dt, cb_sigma=0.05)
    assert_within_tolerance(_run(x, idx, cb, rpc), O.vq_gemm_bl_residual(x, idx, cb, rpc), (M, K, N, v, C, S))


def test_prefill_route_equals_the_dense_product_of_the_dequantised_weights_bit_for_bit():
    # the fused kernel hands the tensor core exactly the rounded W: same bits as dequantise-then-dense when the
    # K loops are not split (no workspace partials): compare through the whole-tile schedule of a small shape
    x, idx, cb = O.make_residual_inputs(256, 512, 512, 8, 256, 128, stages=2, seed=9, cb_sigma=0.05)
    y = V.vq_gemm_residual(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=128)
    w = V.dequant_residual(idx.cuda(), cb.cuda(), rows_per_codebook=128)
    y2 = V.gemm(x.cuda(), w.t().contiguous())
    torch.cuda.synchronize()
    assert float((y.float() - y2.float()).abs().max()) <= 2e-3 * float(y2.float().abs().max())
    # deterministic
    y3 = V.vq_gemm_residual(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=128)
    assert torch.equal(bits(y), bits(y3))


def test_one_stage_is_the_plain_product():
    x, idx, cb = O.make_residual_inputs(4, 1024, 256, 4, 256, 128, stages=1, seed=4)
    a = V.vq_gemm_residual(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=128)
    b = V.vq_gemm(x.cuda(), idx[0].cuda(), cb[0].cuda(), rows_per_codebook=128, layout="bl")
    assert torch.equal(bits(a), bits(b))


def test_argument_checks():
    x, idx, cb = O.make_residual_inputs(4, 256, 64, 4, 256, 0, stages=2, seed=1)
    with pytest.raises(RuntimeError):
        V.vq_gemm_residual(x.cuda(), idx[0].cuda(), cb.cuda())            # indices not [S, N, K/v]
    with pytest.raises(RuntimeError):
        V.vq_gemm_residual(x.cuda(), idx.cuda(), cb[:1].cuda())           # stage counts differ
    with pytest.raises(RuntimeError):
        V.vq_gemm_residual(x, idx, cb)                                    # CPU tensors
