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


def test_misaligned_codebook_is_routed_or_refused_never_faulted():
    """A codebook whose address is not a multiple of its entry size (2v bytes) cannot be read by the kernels
    that fetch whole entries: the automatic route then takes the half-by-half generic kernel, and asking for the
    dequantising route explicitly returns a status code.  (A misaligned-address fault would lose the context.)"""
    import ctypes
    from vq_gemm_b200 import _lib
    lib = _lib.load()
    M, K, N, v, C, rpc = 130, 256, 256, 8, 256, 128
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=5)
    raw = torch.zeros(cb.numel() + 8, dtype=torch.float16, device="cuda")
    cb_off = raw[4:4 + cb.numel()].view(cb.shape)            # 8 bytes past a 16-byte boundary
    cb_off.copy_(cb)
    assert cb_off.data_ptr() % 16 == 8
    xd, idd = x.cuda(), idx.cuda()
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    need = lib.vqg_workspace_bytes(M, N, K, v, C, 1, rpc, 0, _lib.PATH_TWO_PHASE)
    ws_raw = torch.zeros(need + 1024, dtype=torch.uint8, device="cuda")
    ws_ptr = (ws_raw.data_ptr() + 1023) // 1024 * 1024       # workspaces are 1024-byte aligned
    st = lib.vqg_gemm(xd.data_ptr(), idd.data_ptr(), cb_off.data_ptr(), y.data_ptr(), M, N, K, v, C, 1, rpc, 0,
                      ws_ptr, need, s)
    assert st == _lib.OK
    torch.cuda.synchronize()
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, rpc))
    before = lib.vqg_launch_count()
    st = lib.vqg_gemm_path(xd.data_ptr(), idd.data_ptr(), cb_off.data_ptr(), y.data_ptr(), M, N, K, v, C, 1, rpc, 0,
                           _lib.PATH_TWO_PHASE, ws_ptr, need, s)
    assert st == _lib.ERR_BAD_ARG and lib.vqg_launch_count() == before
    assert V.device_status() == 0
