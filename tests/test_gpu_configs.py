"""The five benchmark configurations at full size.  The CPU oracle covers the whole output for the
small ones and a seeded subset of rows and columns for the large ones; the WHOLE output of the large
ones is compared with an fp32 product computed on the device from weights gathered by the (bit-exact)
dequantisation kernel; on top of that, the size-independent properties: bit-exact dequantisation,
determinism, exact linearity under power-of-two scaling of X, and agreement between the fused and the
two-phase route."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits
from vq_gemm_b200.formats import CONFIGS, make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["c1_cpu_ref", "c2_decode", "c3_small_batch"])
def test_small_batch_configs_full_oracle(name):
    s = CONFIGS[name]
    x, idx, cb = make_inputs(s, seed=0)
    y = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=s.rows_per_codebook, layout="bl")
    torch.cuda.synchronize()
    assert V.device_status() == 0
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, s.rows_per_codebook), name)
    y2 = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=s.rows_per_codebook, layout="bl")
    assert torch.equal(bits(y), bits(y2))


@pytest.mark.parametrize("name", ["c4_prefill", "c5_mlp70b"])
def test_large_configs_subset_oracle_and_properties(name):
    s = CONFIGS[name]
    x, idx, cb = make_inputs(s, seed=0)
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    y = V.vq_gemm(xd, idd, cbd, rows_per_codebook=s.rows_per_codebook, layout="bl")
    torch.cuda.synchronize()
    assert V.device_status() == 0
    g = torch.Generator().manual_seed(1)
    rows = torch.randperm(s.M, generator=g)[:64].sort().values
    cols = torch.cat([torch.randperm(s.N, generator=g)[:1024], torch.tensor([0, 127, 128, s.N - 1])]).unique()
    sub = O.vq_gemm_bl_rows(x, idx, cb, s.rows_per_codebook, rows, cols)
    assert_within_tolerance(y.cpu()[rows][:, cols], sub, name)
    # determinism
    y2 = V.vq_gemm(xd, idd, cbd, rows_per_codebook=s.rows_per_codebook, layout="bl")
    assert torch.equal(bits(y), bits(y2))
    # exact linearity under scaling of X by 2
    # (outputs in the fp16 subnormal range round on a fixed grid, so they are compared by distance)
    y4 = V.vq_gemm((xd.float() * 2).half(), idd, cbd, rows_per_codebook=s.rows_per_codebook, layout="bl")
    normal = y.abs() >= 2.0 ** -13
    assert torch.equal((y.float() * 2).half()[normal], y4[normal])
    assert float((y.float() * 2 - y4.float()).abs().max()) <= 2.0 ** -23
    # fused route with whole tiles == dequantise-then-dense route, bit for bit (same operands, same K order);
    # the default route cuts some K loops in two and may differ in the last bits of those tiles
    y3 = V.vq_gemm(xd, idd, cbd, rows_per_codebook=s.rows_per_codebook, layout="bl", path="two_phase")
    y5 = V.vq_gemm(xd, idd, cbd, rows_per_codebook=s.rows_per_codebook, layout="bl", path="tensor_pair")
    assert torch.equal(bits(y5), bits(y3))
    assert float((y.float() - y3.float()).abs().max()) <= 2e-3 * float(y3.float().abs().max())
    assert float((y != y3).float().mean()) < 0.5
    # dequantised weights bit-exact on a slab of rows
    w = V.dequant(idd[:4096], cbd[:32], rows_per_codebook=128).cpu()
    assert torch.equal(bits(w), bits(O.dequant_bl_layout(idx[:4096], cb[:32], 128)))


@pytest.mark.parametrize("name", ["c4_prefill", "c5_mlp70b"])
def test_large_configs_whole_output_against_fp32_product_on_device(name):
    """Every element of Y against torch's fp32 matmul (no TF32) of X and the gathered weights, in column
    blocks of 2048 to bound memory.  The gather is `vqg_dequant`, proven bit-exact against the oracle above
    and in test_gpu_dequant.py; the product is an independent fp32 path.  Same two bounds as the contract:
    max|dY| <= 1e-2 max|Y| and |dY| <= 2e-2 (|Y| + 1) for every element."""
    s = CONFIGS[name]
    x, idx, cb = make_inputs(s, seed=0)
    xd, idd, cbd = x.cuda(), idx.cuda(), cb.cuda()
    y = V.vq_gemm(xd, idd, cbd, rows_per_codebook=s.rows_per_codebook, layout="bl")
    torch.cuda.synchronize()
    assert V.device_status() == 0
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        xf = xd.float()
        rpc, step = s.rows_per_codebook, 2048
        max_abs = ref_max = 0.0
        n_bad = 0
        for n0 in range(0, s.N, step):
            n1 = min(s.N, n0 + step)
            w = V.dequant(idd[n0:n1], cbd[n0 // rpc:(n1 + rpc - 1) // rpc], rows_per_codebook=rpc)
            ref = (xf @ w.float().t()).half().float()
            d = (y[:, n0:n1].float() - ref).abs()
            max_abs = max(max_abs, float(d.max()))
            ref_max = max(ref_max, float(ref.abs().max()))
            n_bad += int((d > O.ELT_TOL * (ref.abs() + 1.0)).sum())
            assert bool(torch.isfinite(y[:, n0:n1]).all())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert n_bad == 0 and max_abs <= O.REL_TOL * ref_max, (name, max_abs, ref_max, n_bad)
