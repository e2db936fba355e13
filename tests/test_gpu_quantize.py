"""Quantiser and packer on the GPU against the CPU restatement: indices and codebooks bit for bit."""
import numpy as np
import pytest
import torch

import vq_gemm_b200 as V
from oracle import quantize_oracle as Q
from vq_gemm_b200 import quantize as VQ

pytestmark = pytest.mark.gpu


def _weights(N, K, seed, sigma=0.05):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * sigma).half()


@pytest.mark.parametrize("N,K,v,C,rpc", [
    (256, 512, 8, 256, 128),
    (256, 256, 4, 256, 128),
    (128, 128, 2, 256, 0),
    (200, 64, 4, 37, 128),       # ragged last group, odd codebook size
    (64, 256, 8, 4096, 0),       # 2-byte indices, single large codebook
    (96, 256, 8, 1024, 0),       # 2-byte indices, codebook that still fits the packed search and the 32-bit counters
    (512, 2048, 4, 256, 128),    # several accumulation rounds per block
])
def test_assign_and_update_match_the_rules_bit_for_bit(N, K, v, C, rpc):
    w = _weights(N, K, seed=N + K + v)
    cb = VQ.initial_codebook(w, v, C, rpc, seed=1)
    wd, cbd = w.cuda(), cb.cuda()
    idx = VQ.assign(wd, cbd, rpc)
    ref_idx = Q.assign(w.numpy(), cb.numpy(), rpc)
    assert idx.cpu().numpy().dtype == ref_idx.dtype
    assert np.array_equal(idx.cpu().numpy(), ref_idx)
    VQ.kmeans_update(wd, idx, cbd, rpc)
    ref_cb = Q.update(w.numpy(), ref_idx, cb.numpy(), rpc)
    assert np.array_equal(cbd.cpu().numpy().view(np.int16), ref_cb.view(np.int16))
    assert V.device_status() == 0


@pytest.mark.parametrize("value", [65504.0, -65504.0, 5.9604645e-08, 0.333251953125])
def test_update_is_exact_at_the_limits_of_its_counters(value):
    # every sub-vector of a group names entry 0 and every weight is the same extreme value: the per-round 32-bit
    # counters of the accumulation reach their largest possible contents (2048 x the largest high part, or the
    # largest low part); the mean must come back as the value itself
    N, K, v, C, rpc = 64, 4096, 4, 256, 64
    w = torch.full((N, K), value, dtype=torch.float16)
    w[1, 5] = -w[1, 5]                                   # one element of the other sign
    idx = torch.zeros(N, K // v, dtype=torch.uint8)
    idx[3, 7] = 9                                        # one sub-vector elsewhere: entry 9 becomes that sub-vector
    cb = torch.zeros(1, C, v, dtype=torch.float16)
    cbd = cb.cuda()
    VQ.kmeans_update(w.cuda(), idx.cuda(), cbd, rpc)
    ref_cb = Q.update(w.numpy(), idx.numpy(), cb.numpy(), rpc)
    assert np.array_equal(cbd.cpu().numpy().view(np.int16), ref_cb.view(np.int16))
    assert float(cbd[0, 9, 0]) == float(w[0, 0]) and V.device_status() == 0


def test_kmeans_pipeline_equals_oracle_and_feeds_the_product():
    N, K, v, C, rpc = 256, 512, 8, 256, 128
    w = _weights(N, K, seed=9)
    idx, cb = VQ.kmeans_quantize(w.cuda(), v=v, entries=C, rows_per_codebook=rpc, iters=4, seed=3)
    # the same loop on the CPU
    rcb = VQ.initial_codebook(w, v, C, rpc, seed=3).numpy()
    ridx = Q.assign(w.numpy(), rcb, rpc)
    errs = [Q.distortion(w.numpy(), ridx, rcb, rpc)]
    for _ in range(4):
        rcb = Q.update(w.numpy(), ridx, rcb, rpc)
        ridx = Q.assign(w.numpy(), rcb, rpc)
        errs.append(Q.distortion(w.numpy(), ridx, rcb, rpc))
    assert np.array_equal(idx.cpu().numpy(), ridx)
    assert np.array_equal(cb.cpu().numpy().view(np.int16), rcb.view(np.int16))
    assert errs[-1] < 0.9 * errs[0]
    # the quantised layer through the product: close to the dense product by the quantisation error only
    x = (torch.randn(32, K, generator=torch.Generator().manual_seed(4))).half().cuda()
    y = V.vq_gemm(x, idx, cb, rows_per_codebook=rpc, layout="bl")
    wq = V.dequant(idx, cb, rows_per_codebook=rpc)
    assert torch.equal(wq.cpu(), torch.from_numpy(rcb.astype(np.float16))[torch.arange(N) // rpc][
        torch.arange(N)[:, None], torch.from_numpy(ridx.astype(np.int64))].reshape(N, K))
    dense = x.float() @ wq.float().t()
    assert float((y.float() - dense).abs().max()) <= 2e-2 * (float(dense.abs().max()) + 1)


def test_idempotence_at_full_size():
    # assigning the dequantised weights gives back weights that dequantise to themselves (size-independent property)
    N, K, v, C, rpc = 4096, 4096, 8, 256, 128
    w = _weights(N, K, seed=5).cuda()
    cb = VQ.initial_codebook(w, v, C, rpc, seed=2)
    idx = VQ.assign(w, cb, rpc)
    wq = V.dequant(idx, cb, rows_per_codebook=rpc)
    idx2 = VQ.assign(wq, cb, rpc)
    assert torch.equal(V.dequant(idx2, cb, rows_per_codebook=rpc), wq)
    # every chosen entry is at least as near as a sample of other entries
    sub = w.reshape(-1, v)[:4096].float()
    g = (torch.arange(4096, device="cuda") // (K // v)) // rpc
    chosen = cb[g, idx.reshape(-1)[:4096].long()].float()
    other = cb[g, torch.randint(0, C, (4096,), device="cuda")].float()
    assert bool((((sub - chosen) ** 2).sum(1) <= ((sub - other) ** 2).sum(1) + 1e-6).all())


def test_pack12_round_trip_and_layout():
    g = torch.Generator().manual_seed(6)
    idx = torch.randint(0, 4096, (1024, 1024), generator=g).to(torch.int16)
    packed = VQ.pack12(idx.cuda())
    assert packed.shape == (1024, 1536)
    assert np.array_equal(packed.cpu().numpy(), Q.pack12(idx.numpy()))
    assert torch.equal(VQ.unpack12(packed).cpu(), idx)
    with pytest.raises(RuntimeError):
        VQ.pack12(idx[:, :3].contiguous().cuda())
    # a count that leaves a tail behind the 16-index groups, and buffers that are only 4-byte aligned (the wide
    # kernels want 16 / 8 bytes and are not used then)
    for n, shift in ((16 * 37 + 6, 0), (16 * 5, 2), (10, 0), (4096, 6)):
        flat = torch.randint(0, 4096, (n + shift,), generator=g).to(torch.int16)
        buf = flat.cuda()
        view = buf[shift:]
        assert view.data_ptr() % 4 == 0
        pk = VQ.pack12(view)
        assert np.array_equal(pk.cpu().numpy(), Q.pack12(flat[shift:].numpy()[None])[0])
        assert torch.equal(VQ.unpack12(pk).cpu(), flat[shift:])


def test_product_enqueued_right_behind_the_quantiser_sees_the_new_weights():
    """The small-batch kernels read indices and codebooks before they wait for the kernel ahead of them on the
    stream; behind the library's own quantiser kernels they are launched in plain stream order instead.  Ten
    rounds of (new assignment, product) with no host synchronisation in between, each checked afterwards."""
    N, K, v, C, rpc, M = 2048, 4096, 4, 256, 128, 2
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(3)).half().cuda()
    outs, idxs = [], []
    cbs = [VQ.initial_codebook(_weights(N, K, seed=20 + i).cuda(), v, C, rpc, seed=i) for i in range(10)]
    ws = [_weights(N, K, seed=40 + i).cuda() for i in range(10)]
    idx = torch.empty((N, K // v), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    for i in range(10):
        VQ.assign(ws[i], cbs[i], rpc, out=idx)                                  # writes the indices ...
        outs.append(V.vq_gemm(x, idx, cbs[i], rows_per_codebook=rpc, layout="bl"))   # ... the product reads them at once
        idxs.append(idx.clone())
    torch.cuda.synchronize()
    for i in range(10):
        want = V.vq_gemm(x, idxs[i], cbs[i], rows_per_codebook=rpc, layout="bl")
        assert torch.equal(outs[i].view(torch.int16), want.view(torch.int16)), i
