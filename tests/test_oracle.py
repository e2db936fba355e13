"""CPU checks of the oracle itself: against the fixtures made by the reference's own gather code
(tests/golden/make_golden.py), against the scalar-loop statement of both rules, and of the
tolerance checker."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import vq_oracle as O


def _load(path):
    z = np.load(path)
    return {k: torch.from_numpy(z[k]) for k in z.files}


@pytest.mark.parametrize("tag", ["ref_small", "ref_two_tiles", "ref_ragged", "ref_nq4_bridge"])
def test_ref_layout_matches_reference_gather(golden_dir, tag):
    g = _load(os.path.join(golden_dir, tag + ".npz"))
    wdec = O.dequant_ref_layout(g["w"], g["codebook"])
    assert torch.equal(wdec.view(torch.int16), g["w_decoded"].view(torch.int16))  # bit-exact
    y = O.vq_gemm_ref_layout(g["x"], g["w"], g["codebook"])
    assert torch.equal(y.view(torch.int16), g["y"].view(torch.int16))


@pytest.mark.parametrize("tag", ["bl_v4_c256_groups", "bl_v8_c4096_single", "bl_v8_c256_groups"])
def test_bl_layout_matches_fixture(golden_dir, tag):
    g = _load(os.path.join(golden_dir, tag + ".npz"))
    M, K, N, v, C, rpc, seed = [int(t) for t in g["meta"]]
    wdec = O.dequant_bl_layout(g["idx"], g["codebook"], rpc)
    assert torch.equal(wdec.view(torch.int16), g["w_decoded"].view(torch.int16))
    y = O.vq_gemm_bl(g["x"], g["idx"], g["codebook"], rpc)
    assert O.check_tolerance(y, g["y"])["ok"]
    assert (y.float() - g["y"].float()).abs().max() <= 2e-3  # same algorithm; only summation order may differ


def test_bl_gather_matches_bytes_gathered_by_the_reference(golden_dir):
    """With Nq = 4 the reference's gather (bench.py:46-55) uses one codebook for every index column, and its
    w_decoded [K, 8] is the generalised rule applied to idx = w read as [N = K, 4], v = 2, single codebook:
    the BL gather against bytes produced by the reference's own code."""
    g = _load(os.path.join(golden_dir, "ref_nq4_bridge.npz"))
    assert g["w"].shape[1] == 4 and g["codebook"].shape[0] == 1
    a = O.dequant_bl_layout(g["w"], g["codebook"][0], 0)
    assert a.shape == g["w_decoded"].shape
    assert torch.equal(a.view(torch.int16), g["w_decoded"].view(torch.int16))
    b = O.dequant_bl_scalar(g["w"][:64], g["codebook"][0], 0)
    assert torch.equal(b.view(torch.int16), g["w_decoded"][:64].view(torch.int16))


def test_packed_index_fixture(golden_dir):
    """The fixture's packed bytes (written byte by byte by its generator) against the numpy packer, both ways, and
    the weights behind them."""
    from oracle import quantize_oracle as Q
    g = _load(os.path.join(golden_dir, "bl_v8_c4096_packed12.npz"))
    assert np.array_equal(Q.pack12(g["idx"].numpy()), g["packed"].numpy())
    assert np.array_equal(Q.unpack12(g["packed"].numpy()), g["idx"].numpy())
    wdec = O.dequant_bl_layout(torch.from_numpy(Q.unpack12(g["packed"].numpy())), g["codebook"], 0)
    assert torch.equal(wdec.view(torch.int16), g["w_decoded"].view(torch.int16))


def test_golden_files_all_covered(golden_dir):
    tags = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(golden_dir, "*.npz")))
    assert tags == ["bl_residual_v8_c256_s2", "bl_v4_c256_groups", "bl_v8_c256_groups", "bl_v8_c4096_packed12",
                    "bl_v8_c4096_single", "ref_nq4_bridge", "ref_ragged", "ref_small", "ref_two_tiles"]


@pytest.mark.parametrize("N,K,v,C,rpc,dtype", [
    (32, 16, 4, 256, 16, torch.uint8),
    (6, 24, 8, 300, 0, torch.int16),
    (20, 8, 2, 7, 5, torch.uint8),
])
def test_bl_vectorised_equals_scalar_rule(N, K, v, C, rpc, dtype):
    _, idx, cb = O.make_bl_inputs(1, K, N, v, C, rpc, seed=N + K, idx_dtype=dtype)
    a = O.dequant_bl_layout(idx, cb, rpc)
    b = O.dequant_bl_scalar(idx, cb, rpc)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_ref_vectorised_equals_scalar_rule():
    _, w, cb = O.make_ref_inputs(1, 12, 16, seed=5)
    assert torch.equal(O.dequant_ref_layout(w, cb).view(torch.int16), O.dequant_ref_scalar(w, cb).view(torch.int16))


def test_uint16_indices_above_32767_are_unsigned():
    cb = (torch.arange(40000 * 2).reshape(1, 40000, 2) % 2048).half()
    idx = torch.tensor([[39999, 5]], dtype=torch.int32).to(torch.int16)  # 39999 wraps negative in int16
    w = O.dequant_bl_layout(idx, cb, 0)
    assert torch.equal(w[0, :2], cb[0, 39999]) and torch.equal(w[0, 2:], cb[0, 5])


def test_subset_oracle_equals_full():
    x, idx, cb = O.make_bl_inputs(8, 64, 256, 4, 256, 128, seed=9)
    full = O.vq_gemm_bl(x, idx, cb, 128)
    rows = torch.tensor([0, 3, 7])
    cols = torch.tensor([1, 127, 128, 255])
    sub = O.vq_gemm_bl_rows(x, idx, cb, 128, rows, cols)
    assert torch.equal(sub, full[rows][:, cols])


def test_tolerance_checker():
    y = torch.randn(64, 64).half()
    assert O.check_tolerance(y, y)["ok"]
    bad = y.clone()
    bad[3, 4] += 1.0
    r = O.check_tolerance(bad, y)
    assert not r["ok"] and r["n_bad"] == 1
    assert not O.check_tolerance(torch.full_like(y, float("nan")), y)["ok"]
    assert not O.check_tolerance(y[:8], y)["ok"]
    assert O.check_tolerance(torch.empty(0, 4), torch.empty(0, 4))["ok"]


def test_empty_shapes():
    x, idx, cb = O.make_bl_inputs(0, 16, 8, 4, 256, 0, seed=0)
    assert O.vq_gemm_bl(x, idx, cb, 0).shape == (0, 8)
    x, idx, cb = O.make_bl_inputs(4, 0, 8, 4, 256, 0, seed=0)
    y = O.vq_gemm_bl(x, idx, cb, 0)
    assert y.shape == (4, 8) and float(y.abs().max()) == 0.0


def test_residual_rule_vectorised_equals_scalar_and_fixture(golden_dir):
    g = _load(os.path.join(golden_dir, "bl_residual_v8_c256_s2.npz"))
    M, K, N, v, C, rpc, stages, seed = [int(t) for t in g["meta"]]
    w = O.dequant_bl_residual(g["idx"], g["codebook"], rpc)
    assert torch.equal(w.view(torch.int16), g["w_decoded"].view(torch.int16))
    # one stage is the plain format; two equal stages double every weight exactly
    assert torch.equal(O.dequant_bl_residual(g["idx"][:1], g["codebook"][:1], rpc).view(torch.int16),
                       O.dequant_bl_layout(g["idx"][0], g["codebook"][0], rpc).view(torch.int16))
    _, idx, cb = O.make_residual_inputs(1, 32, 24, 4, 37, 8, stages=3, seed=2)
    assert torch.equal(O.dequant_bl_residual(idx, cb, 8).view(torch.int16),
                       O.dequant_bl_residual_scalar(idx, cb, 8).view(torch.int16))
    y = O.vq_gemm_bl_residual(g["x"], g["idx"], g["codebook"], rpc)
    assert O.check_tolerance(y, g["y"])["ok"]
