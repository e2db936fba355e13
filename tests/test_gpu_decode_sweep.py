"""Seeded sweep of small shapes through the M <= 16 kernel: every batch size, short and long K (one or several
chunks, K a multiple of 256 but not always of 512), N down to a single 8-row unit and not always a whole tile,
all three (v, index width) combinations, grouped and single codebooks, replicated and unreplicated images."""
import random

import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, run_bl

pytestmark = pytest.mark.gpu


def _cases():
    rnd = random.Random(20240607)
    out = []
    for i in range(72):
        M = rnd.choice([1, 2, 3, 4, 5, 7, 8, 9, 12, 16])
        v, dt, C = rnd.choice([(4, torch.uint8, 256), (4, torch.uint8, 37), (8, torch.uint8, 256), (8, torch.int16, 300),
                               (8, torch.int16, 4096)])
        K = 256 * rnd.choice([1, 2, 3, 4, 5, 8, 16, 17, 20, 33])
        rpc = rnd.choice([0, 0, 16, 32, 48, 128])
        if rpc:
            N = rpc * rnd.choice([1, 2, 3, 5])
        else:
            N = 8 * rnd.choice([1, 2, 3, 5, 8, 13, 30])
        out.append((M, K, N, v, C, rpc, dt))
    return out


@pytest.mark.parametrize("M,K,N,v,C,rpc,dt", _cases())
def test_decode_sweep(M, K, N, v, C, rpc, dt):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=M * 1009 + K + N, idx_dtype=dt, cb_sigma=0.05)
    from vq_gemm_b200 import _lib
    ib = 1 if dt == torch.uint8 else 2
    # every shape of this sweep is inside the kernel's rules (K % 256 == 0, N % 8 == 0, whole tiles per group)
    y = run_bl(V, x, idx, cb, rpc, path="decode")
    assert_within_tolerance(y, O.vq_gemm_bl(x, idx, cb, rpc), (M, K, N, v, C, rpc))
    need = _lib.load().vqg_workspace_bytes(M, N, K, v, C, ib, rpc, _lib.LAYOUT_BL, _lib.PATH_DECODE)
    assert need == 0 or K > 4096          # scratch only when K is split over CTAs
