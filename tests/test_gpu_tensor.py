"""The tcgen05 / TMEM / TMA kernels against the oracle: dense operand variant, fused-dequant
variant, and the two-phase route (dequantise, then dense)."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits, load_golden, run_bl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (128, 256, 256), (256, 512, 512), (100, 128, 96), (300, 1024, 1280)])
def test_dense_gemm(M, K, N):
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g).half()
    w = (torch.randn(K, N, generator=g) * 0.1).half()
    y = V.gemm(x.cuda(), w.cuda()).cpu()
    assert V.device_status() == 0
    assert_within_tolerance(y, (x.float() @ w.float()).half())


@pytest.mark.parametrize("M,K,N,v,rpc", [
    (128, 64, 256, 4, 128),       # one tile, one K step
    (128, 256, 256, 4, 128),      # one tile, wraps the 3-stage ring
    (128, 512, 256, 8, 128),      # v = 8
    (256, 1024, 512, 4, 128),     # 4 tiles
    (200, 512, 384, 4, 128),      # ragged M, N = 1.5 tiles
    (130, 128, 256, 8, 128),      # golden-sized
    (64, 2048, 128, 4, 0),        # single codebook, half tile
    (1024, 1024, 2048, 8, 256),   # 256 rows per codebook, many tiles per CTA? (64 tiles)
    (4096, 512, 4864, 4, 128),    # more tiles than SMs: persistent loop + accumulator ping-pong
])
@pytest.mark.parametrize("path", ["tensor", "tensor_pair", "tensor_ts"])
def test_fused_matches_oracle(M, K, N, v, rpc, path):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, rpc, seed=M + K + N + v, cb_sigma=0.05)
    if path == "tensor_ts" and K % 128:   # that kernel's pipeline stage is 128 K values
        with pytest.raises(RuntimeError, match="unsupported"):
            run_bl(V, x, idx, cb, rpc, path=path)
        return
    y = run_bl(V, x, idx, cb, rpc, path=path)
    assert_within_tolerance(y, O.vq_gemm_bl(x, idx, cb, rpc))


def test_fused_small_codebook():
    x, idx, cb = O.make_bl_inputs(128, 256, 256, 4, 37, 128, seed=2, cb_sigma=0.05)
    assert_within_tolerance(run_bl(V, x, idx, cb, 128, path="tensor"), O.vq_gemm_bl(x, idx, cb, 128))


def test_golden_fixture_through_tensor_path():
    g = load_golden("bl_v8_c256_groups")
    y = run_bl(V, g["x"], g["idx"], g["codebook"], 128, path="tensor")
    assert_within_tolerance(y, g["y"])


@pytest.mark.parametrize("M,K,N,v,C,rpc,dt", [
    (256, 512, 512, 4, 256, 128, torch.uint8),
    (128, 256, 256, 8, 4096, 0, torch.int16),
])
def test_two_phase(M, K, N, v, C, rpc, dt):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=3, idx_dtype=dt, cb_sigma=0.05)
    y = run_bl(V, x, idx, cb, rpc, path="two_phase")
    assert_within_tolerance(y, O.vq_gemm_bl(x, idx, cb, rpc))


@pytest.mark.parametrize("tag,path", [("ref_small", "two_phase"), ("ref_small", "auto"), ("ref_two_tiles", "auto")])
def test_reference_format(tag, path):
    # ref_two_tiles has K = 96 (not a multiple of 64): auto routes it to the generic kernel
    g = load_golden(tag)
    y = V.vq_gemm(g["x"].cuda(), g["w"].cuda(), g["codebook"].cuda(), layout="ref", path=path).cpu()
    assert V.device_status() == 0
    assert_within_tolerance(y, g["y"], tag)


def test_fused_deterministic():
    x, idx, cb = O.make_bl_inputs(512, 1024, 1024, 4, 256, 128, seed=8)
    xs, ids, cbs = x.cuda(), idx.cuda(), cb.cuda()
    outs = [V.vq_gemm(xs, ids, cbs, layout="bl", path="tensor").cpu() for _ in range(5)]
    for o in outs[1:]:
        assert torch.equal(bits(outs[0]), bits(o))
    assert V.device_status() == 0


def test_pair_kernel_equals_single_cta_kernel_bitwise():
    # same operands, same K order inside every accumulator -> same bits
    x, idx, cb = O.make_bl_inputs(700, 1024, 1280, 4, 256, 128, seed=12)
    a = run_bl(V, x, idx, cb, 128, path="tensor")
    b = run_bl(V, x, idx, cb, 128, path="tensor_pair")
    assert torch.equal(bits(a), bits(b))
    outs = [run_bl(V, x, idx, cb, 128, path="tensor_pair") for _ in range(3)]
    for o in outs:
        assert torch.equal(bits(o), bits(b))


def test_tensor_memory_operand_kernel_is_deterministic_and_close_to_the_others():
    # weights as the MMA's tensor-memory operand, problem transposed inside the kernel
    x, idx, cb = O.make_bl_inputs(700, 1024, 1280, 4, 256, 128, seed=12)
    ref = O.vq_gemm_bl(x, idx, cb, 128)
    outs = [run_bl(V, x, idx, cb, 128, path="tensor_ts") for _ in range(3)]
    assert_within_tolerance(outs[0], ref)
    for o in outs[1:]:
        assert torch.equal(bits(o), bits(outs[0]))
    b = run_bl(V, x, idx, cb, 128, path="tensor_pair")
    assert float((outs[0].float() - b.float()).abs().max()) <= 2e-3 * float(ref.float().abs().max())


def test_fused_equals_two_phase_bitwise():
    # both routes feed identical fp16 operands to the same MMA sequence
    x, idx, cb = O.make_bl_inputs(256, 512, 512, 8, 256, 128, seed=10)
    a = run_bl(V, x, idx, cb, 128, path="tensor")
    b = run_bl(V, x, idx, cb, 128, path="two_phase")
    assert torch.equal(bits(a), bits(b))


@pytest.mark.parametrize("M,K,N,v", [
    (700, 2048, 1024, 4),     # 12 tiles x 8 units over 74 CTA pairs: tiles shared by up to 8 pairs
    (520, 4096, 768, 8),      # 9 tiles x 8 units: one unit per pair
    (1024, 4096, 2304, 8),    # 288 units: every pair ends in the middle of a tile
])
def test_even_split_of_k_loops_matches_whole_tiles(M, K, N, v):
    # with a workspace the K loops are dealt out evenly over the CTA pairs and shared tiles are summed
    # from fp32 partials in pair order; without one every tile is computed by a single pair
    import ctypes
    from vq_gemm_b200 import _lib
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, 128, seed=M + N, cb_sigma=0.05)
    ref = O.vq_gemm_bl(x, idx, cb, 128)
    outs = [run_bl(V, x, idx, cb, 128, path="tensor_ts") for _ in range(3)]
    assert_within_tolerance(outs[0], ref)
    for o in outs[1:]:
        assert torch.equal(bits(o), bits(outs[0]))      # the counters are back at zero; order is fixed
    lib = _lib.load()
    assert lib.vqg_workspace_bytes(M, N, K, v, 256, 1, 128, 0, _lib.PATHS["tensor_ts"]) > lib.vqg_workspace_counter_bytes()
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    y = torch.empty(M, N, dtype=torch.float16, device="cuda")
    st = lib.vqg_gemm_path(xd.data_ptr(), idd.data_ptr(), cbd.data_ptr(), y.data_ptr(), M, N, K, v, 256, 1, 128, 0,
                           _lib.PATHS["tensor_ts"], None, 0, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert V.device_status() == 0
    assert_within_tolerance(y.cpu(), ref)
    # the two schedules round differently only in the last fp32 bits of the partial sums
    assert float((y.cpu().float() - outs[0].float()).abs().max()) <= 2e-3 * float(ref.float().abs().max())
