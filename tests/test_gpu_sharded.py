"""N-sharded mode on real GPUs: with 2 ranks, both ways of assembling Y (fused peer stores over
NVLink, NCCL all-gather + re-layout) must equal the single-GPU result bit for bit.  Runs as child
processes; skipped on a single-GPU box (the world-size-1 path is covered below)."""
import os
import subprocess
import sys

import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import ROOT, assert_within_tolerance, bits

pytestmark = pytest.mark.gpu


def test_world_size_one_is_the_plain_product():
    import ctypes
    from vq_gemm_b200 import _lib
    x, idx, cb = O.make_bl_inputs(130, 256, 512, 4, 256, 128, seed=2)
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    y = torch.zeros(130, 512, dtype=torch.float16, device="cuda")
    arr = (ctypes.c_void_p * 1)(y.data_ptr())
    st = _lib.load().vqg_gemm_sharded(xd.data_ptr(), idd.data_ptr(), cbd.data_ptr(), arr, 0, 1, 130, 512, 256, 4, 256, 1,
                                      128, None, 0, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert torch.equal(bits(y), bits(V.vq_gemm(xd, idd, cbd, rows_per_codebook=128, layout="bl")))
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, 128))


def test_column_block_with_leading_dimension():
    # a rank's block written into a wider Y (emulates rank 1 of 2 on one GPU, no peers)
    import ctypes
    from vq_gemm_b200 import _lib
    x, idx, cb = O.make_bl_inputs(64, 512, 512, 8, 256, 128, seed=3)
    full = O.vq_gemm_bl(x, idx, cb, 128)
    y = torch.zeros(64, 512, dtype=torch.float16, device="cuda")
    other = torch.zeros_like(y)
    # the workspace a rank's block needs, as the header tells callers to size it (zeroed once)
    nbytes = _lib.load().vqg_workspace_bytes(64, 256, 512, 8, 256, 1, 128, 0, 0)
    ws = torch.zeros(max(nbytes, 1), dtype=torch.uint8, device="cuda")
    for rank in range(2):
        idx_l, cb_l = idx[rank * 256:(rank + 1) * 256].contiguous().cuda(), cb[rank * 2:(rank + 1) * 2].contiguous().cuda()
        ptrs = [other.data_ptr(), other.data_ptr()]
        ptrs[rank] = y.data_ptr()
        arr = (ctypes.c_void_p * 2)(*ptrs)
        st = _lib.load().vqg_gemm_sharded(x.cuda().data_ptr(), idx_l.data_ptr(), cb_l.data_ptr(), arr, rank, 2, 64, 256, 512,
                                          8, 256, 1, 128, ws.data_ptr() if nbytes else None, nbytes,
                                          torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()
    # y holds both blocks (each call wrote its own block locally); `other` received both as the "peer"
    assert_within_tolerance(y.cpu(), full)
    assert torch.equal(bits(y), bits(other))


@pytest.mark.parametrize("M,K,N,v,rpc,slabs", [
    (2048, 1024, 2048, 8, 128, (512, 1536)),     # prefill kernel, a small first slab and the rest
    (64, 512, 1024, 4, 128, (256, 256, 512)),
    (8, 512, 768, 8, 0, (256, 512)),             # single codebook: every slab uses the same one
])
def test_column_slabs_of_one_block(M, K, N, v, rpc, slabs):
    # vqg_gemm_sharded_cols: the block handed over in column slabs with its own leading dimension and a "peer"
    # copy; every slab equals the stand-alone product of the same columns bit for bit
    import ctypes
    from vq_gemm_b200 import _lib
    lib = _lib.load()
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, rpc, seed=M + N)
    xd = x.cuda()
    y = torch.zeros(M, N + 64, dtype=torch.float16, device="cuda")     # wider than the block: ld_y = N + 64, col0 = 32
    peer = torch.zeros_like(y)
    arr = (ctypes.c_void_p * 2)(y.data_ptr(), peer.data_ptr())
    nbytes = max(lib.vqg_workspace_bytes(M, n, K, v, 256, 1, rpc, 0, 0) for n in slabs)
    ws = torch.zeros(max(nbytes, 1), dtype=torch.uint8, device="cuda")
    c0 = 0
    for n in slabs:
        idx_s = idx[c0:c0 + n].contiguous().cuda()
        cb_s = (cb[c0 // rpc:(c0 + n) // rpc] if rpc else cb).contiguous().cuda()
        st = lib.vqg_gemm_sharded_cols(xd.data_ptr(), idx_s.data_ptr(), cb_s.data_ptr(), arr, None, 0, 2, M, n, K, v, 256, 1, rpc,
                                       32 + c0, N + 64, ws.data_ptr() if nbytes else None, nbytes,
                                       torch.cuda.current_stream().cuda_stream)
        assert st == 0
        alone = V.vq_gemm(xd, idx_s, cb_s, rows_per_codebook=rpc, layout="bl")
        torch.cuda.synchronize()
        assert torch.equal(bits(y[:, 32 + c0:32 + c0 + n]), bits(alone))
        c0 += n
    assert torch.equal(bits(y), bits(peer))
    assert float(y[:, :32].abs().max()) == 0 and float(y[:, 32 + N:].abs().max()) == 0     # nothing outside the block
    assert_within_tolerance(y[:, 32:32 + N].cpu(), O.vq_gemm_bl(x, idx, cb, rpc))
    bad = lib.vqg_gemm_sharded_cols(xd.data_ptr(), idx_s.data_ptr(), cb_s.data_ptr(), arr, None, 0, 2, M, n, K, v, 256, 1, rpc,
                                    N, N + 64, None, 0, None)
    assert bad == _lib.ERR_BAD_ARG                                      # the slab would run past the leading dimension


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_ranks_gather_through_the_switch_equals_single_gpu():
    # the multimem-store epilogue (NVLS multicast mapping of the symmetric buffers), where the fabric offers it;
    # both ranks run to the end (a rank must not leave while its memory is bound to the multicast object)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", VQG_WORKER_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29513", os.path.join(ROOT, "tests", "_sharded_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert p.returncode == 0 and "SHARDED_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
    if "MULTICAST_TESTED" not in p.stdout:
        pytest.skip("no multicast mapping on this machine: only the peer-store and NCCL modes ran")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_ranks_equal_single_gpu():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29511", os.path.join(ROOT, "tests", "_sharded_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert p.returncode == 0 and "SHARDED_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_prefill_kernel_writes_every_rank_buffer():
    # three ranks emulated on one GPU: the prefill kernel stores its block into its own buffer and into the
    # two others (rows beyond M = 300 and columns beyond the block's edge are not touched)
    import ctypes
    from vq_gemm_b200 import _lib
    M, K, N, G = 300, 1024, 1536, 3
    x, idx, cb = O.make_bl_inputs(M, K, N, 8, 256, 128, seed=8)
    full = O.vq_gemm_bl(x, idx, cb, 128)
    bufs = [torch.full((M + 4, N), 7.0, dtype=torch.float16, device="cuda") for _ in range(G)]   # 4 guard rows
    lib = _lib.load()
    n_local = N // G
    nbytes = lib.vqg_workspace_bytes(M, n_local, K, 8, 256, 1, 128, 0, 0)
    ws = torch.zeros(max(nbytes, 1), dtype=torch.uint8, device="cuda")
    xd = x.cuda()
    for rank in range(G):
        idx_l = idx[rank * n_local:(rank + 1) * n_local].contiguous().cuda()
        cb_l = cb[rank * n_local // 128:(rank + 1) * n_local // 128].contiguous().cuda()
        arr = (ctypes.c_void_p * G)(*[b.data_ptr() for b in bufs])
        st = lib.vqg_gemm_sharded(xd.data_ptr(), idx_l.data_ptr(), cb_l.data_ptr(), arr, rank, G, M, n_local, K, 8, 256, 1, 128,
                                  ws.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()
    assert V.device_status() == 0
    assert_within_tolerance(bufs[0][:M].cpu(), full)
    for b in bufs[1:]:
        assert torch.equal(bits(b[:M]), bits(bufs[0][:M]))
    for b in bufs:
        assert bool((b[M:] == 7.0).all())        # nothing written past row M


@pytest.mark.parametrize("M,K,N,v", [
    (300, 2048, 512, 8),      # prefill kernel: tiles stored to their owners with TMA tensor stores
    (40, 2048, 512, 4),       # small shapes: product into scratch, then the scatter kernel
])
def test_row_parallel_two_ranks_emulated_on_one_gpu(M, K, N, v):
    # rank r multiplies its K slice and writes block o of its partial to slot r of owner o; each owner sums
    import ctypes
    from vq_gemm_b200 import _lib
    from vq_gemm_b200.sharded import shard_weights_k
    G = 2
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, 128, seed=21)
    full = O.vq_gemm_bl(x, idx, cb, 128)
    lib = _lib.load()
    nl, kl = N // G, K // G
    parts = [torch.full((G, M, nl), 9.0, dtype=torch.float16, device="cuda") for _ in range(G)]   # owner o's slots
    cbd = cb.cuda()
    nbytes = lib.vqg_rowparallel_workspace_bytes(M, N, kl, v, 256, 1, 128)
    ws = torch.zeros(max(nbytes, 1), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(G):
        xl = x[:, r * kl:(r + 1) * kl].contiguous().cuda()
        il = shard_weights_k(idx, G, r).cuda()
        arr = (ctypes.c_void_p * G)(*[parts[o][r].data_ptr() for o in range(G)])
        st = lib.vqg_gemm_rowparallel(xl.data_ptr(), il.data_ptr(), cbd.data_ptr(), arr, G, M, N, kl, v, 256, 1, 128,
                                      ws.data_ptr() if nbytes else None, nbytes, stream)
        assert st == 0
        torch.cuda.synchronize()
    assert V.device_status() == 0
    ys = []
    for o in range(G):
        y = torch.empty(M, nl, dtype=torch.float16, device="cuda")
        assert lib.vqg_reduce_slots(parts[o].data_ptr(), y.data_ptr(), G, M, nl, nl, stream) == 0
        ys.append(y)
    torch.cuda.synchronize()
    assert_within_tolerance(torch.cat(ys, dim=1).cpu(), full)
    # slot sums are exactly the fp32 sum of the fp16 partials, in slot order
    want = (parts[0][0].float() + parts[0][1].float()).half()
    assert torch.equal(bits(ys[0]), bits(want))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_row_parallel_two_ranks_over_nvlink():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", VQG_WORKER_MODE="rowparallel")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29512", os.path.join(ROOT, "tests", "_sharded_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert p.returncode == 0 and "SHARDED_OK" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
