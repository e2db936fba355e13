"""CPU checks of the quantiser's restated rules (no GPU): known answers worked out by hand, the
packing round trip, and argument checks of the C entry points that run before any CUDA call."""
import ctypes

import numpy as np
import pytest

from oracle import quantize_oracle as Q


def test_assign_known_answers_and_tie_rule():
    cb = np.array([[[0, 0], [1, 1], [1, 1], [-2, 0.5]]], dtype=np.float16)           # entries 1 and 2 are equal
    w = np.array([[0.1, -0.1, 0.9, 1.2], [-1.5, 0.25, 0.5, 0.5]], dtype=np.float16)
    idx = Q.assign(w, cb, 0)
    # (0.1,-0.1)->0; (0.9,1.2)->1 (lowest of the twins); (-1.5,0.25)->3; (0.5,0.5): d0 = d1 = 0.5 -> 0
    assert idx.tolist() == [[0, 1], [3, 0]]
    assert idx.dtype == np.uint8


def test_update_is_the_exact_mean_and_keeps_unused_entries():
    cb = np.array([[[9, 9], [7, 7], [5, 5]]], dtype=np.float16)
    w = np.array([[1, 2, 3, 4], [0.5, 0.25, 2 ** -24, -1]], dtype=np.float16)
    idx = np.array([[0, 0], [0, 2]], dtype=np.uint8)
    new = Q.update(w, idx, cb, 0)
    assert new[0, 1].tolist() == [7, 7]                                               # nobody chose entry 1
    assert new[0, 2].tolist() == [np.float16(2 ** -24), -1]
    assert new[0, 0].tolist() == [np.float16(4.5 / 3), np.float16(6.25 / 3)]


def test_groups_use_their_own_codebooks():
    rng = np.random.default_rng(0)
    w = rng.standard_normal((8, 16)).astype(np.float16)
    cb = rng.standard_normal((2, 16, 4)).astype(np.float16)
    idx = Q.assign(w, cb, 4)
    assert np.array_equal(idx[:4], Q.assign(w[:4], cb[:1], 0))
    assert np.array_equal(idx[4:], Q.assign(w[4:], cb[1:], 0))


def test_pack12_layout_and_round_trip():
    assert Q.pack12(np.array([[0xABC, 0x123]], dtype=np.int16)).tolist() == [[0xBC, 0x3A, 0x12]]
    rng = np.random.default_rng(1)
    idx = rng.integers(0, 4096, size=(5, 64)).astype(np.int16)
    p = Q.pack12(idx)
    assert p.shape == (5, 96) and p.dtype == np.uint8
    assert np.array_equal(Q.unpack12(p), idx)


def test_lloyd_steps_do_not_raise_distortion_beyond_rounding():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((32, 64)) * 0.05).astype(np.float16)
    cb = w.reshape(-1, 4)[rng.integers(0, 32 * 16, size=16)].reshape(1, 16, 4).copy()
    idx = Q.assign(w, cb, 0)
    errs = [Q.distortion(w, idx, cb, 0)]
    for _ in range(5):
        cb = Q.update(w, idx, cb, 0)
        idx = Q.assign(w, cb, 0)
        errs.append(Q.distortion(w, idx, cb, 0))
    assert errs[-1] < errs[0]
    assert all(b <= a * (1 + 1e-3) for a, b in zip(errs, errs[1:]))


def test_entry_points_reject_bad_arguments_without_cuda():
    from vq_gemm_b200 import _lib
    from vq_gemm_b200.build import build
    build()
    lib = _lib.load()
    p = ctypes.c_void_p(4096)
    assert lib.vqg_quantize_assign(None, p, p, 4, 8, 4, 256, 1, 0, None) == _lib.ERR_BAD_ARG
    assert lib.vqg_quantize_assign(p, p, p, 4, 8, 3, 256, 1, 0, None) == _lib.ERR_UNSUPPORTED       # v
    assert lib.vqg_quantize_assign(p, p, p, 4, 8, 4, 4096, 1, 0, None) == _lib.ERR_UNSUPPORTED     # C vs index width
    assert lib.vqg_quantize_assign(p, p, p, 0, 8, 4, 256, 1, 0, None) == _lib.OK                    # empty
    assert lib.vqg_quantize_update(p, p, p, None, 0, 4, 8, 4, 256, 1, 0, None) == _lib.ERR_WORKSPACE
    assert lib.vqg_quantize_workspace_bytes(256, 8, 256, 128) == 2 * 256 * (8 * 8 + 4)
    assert lib.vqg_pack12(p, p, 3, None) == _lib.ERR_BAD_ARG                                         # odd count
    assert lib.vqg_pack12(p, p, 0, None) == _lib.OK
