"""A bounded device-side wait that runs out: the kernel returns, the host reads a status code, the
device stays usable.  The wait is on a barrier nobody signals, limited to ~10 ms; nothing faults."""
import ctypes

import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance
from vq_gemm_b200 import _lib

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_reports_and_leaves_the_device_usable():
    lib = _lib.load()
    torch.cuda.synchronize()
    assert V.device_status() == 0
    st = lib.vqg_selftest_bounded_wait(20_000_000, torch.cuda.current_stream().cuda_stream)   # ~10 ms
    assert st == 0
    code = ctypes.c_int(-1)
    rc = lib.vqg_device_status(ctypes.byref(code))
    assert rc == _lib.ERR_DEVICE_TIMEOUT and code.value == 10
    assert "wait" in _lib.status_string(rc)
    # the word is cleared by the read, and the context is intact: an ordinary product still works
    assert V.device_status() == 0
    x, idx, cb = O.make_bl_inputs(256, 512, 512, 8, 256, 128, seed=1)
    y = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=128, layout="bl")
    torch.cuda.synchronize()
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, 128))
    assert V.device_status() == 0


def test_limit_is_checked_on_the_host():
    lib = _lib.load()
    assert lib.vqg_selftest_bounded_wait(10, None) == _lib.ERR_BAD_ARG
    assert lib.vqg_selftest_bounded_wait(10**12, None) == _lib.ERR_BAD_ARG
