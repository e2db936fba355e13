"""Helpers shared by the GPU parity tests."""
import os

import numpy as np
import torch

from oracle import vq_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_golden(tag):
    z = np.load(os.path.join(ROOT, "tests", "golden", tag + ".npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def bits(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().contiguous().view(torch.int16)


def assert_within_tolerance(y, y_ref, what=""):
    r = O.check_tolerance(y, y_ref)
    assert r["ok"], f"{what}: {r}"
    return r


def run_bl(V, x, idx, cb, rpc, path="auto"):
    y = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=rpc, layout="bl", path=path)
    torch.cuda.synchronize()
    assert V.device_status() == 0
    return y.cpu()
