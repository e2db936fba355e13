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


def _flag_arrays(n):
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(n)]
    arr = (ctypes.c_void_p * n)(*[f.data_ptr() for f in flags])
    return flags, arr


def test_rank_barrier_with_all_flags_local_passes_and_signals_every_rank():
    """Four ranks emulated on one GPU: the arrivals of the three others are written beforehand (barriers of
    different ranks must not wait for one another as separate launches on one GPU), rank 1 then passes and has
    announced itself in every other rank's array."""
    lib = _lib.load()
    G, me, epoch = 4, 1, 7
    flags, arr = _flag_arrays(G)
    flags[me][:G] = epoch            # everyone has arrived at barrier 7 ...
    flags[me][3] = epoch + 1         # ... and rank 3 is already one barrier ahead, which must not matter
    s = torch.cuda.current_stream().cuda_stream
    assert lib.vqg_rank_barrier(arr, me, G, epoch, 20_000_000, s) == _lib.OK
    torch.cuda.synchronize()
    assert V.device_status() == 0
    for r in range(G):
        if r != me:
            assert int(flags[r][me]) == epoch
            assert int(flags[r].sum()) == epoch      # nothing else written
    # one rank: nothing to do, nothing launched
    before = lib.vqg_launch_count()
    assert lib.vqg_rank_barrier(arr, 0, 1, 1, 20_000_000, s) == _lib.OK
    assert lib.vqg_launch_count() == before


def test_rank_barrier_gives_up_on_a_rank_that_never_arrives():
    """Rank 2's arrival is never written: after ~10 ms the barrier kernel returns with code 11 in the status
    word; the product still runs afterwards."""
    lib = _lib.load()
    G, me, epoch = 3, 0, 1
    flags, arr = _flag_arrays(G)
    flags[me][1] = epoch             # rank 1 arrived, rank 2 did not
    s = torch.cuda.current_stream().cuda_stream
    assert lib.vqg_rank_barrier(arr, me, G, epoch, 20_000_000, s) == _lib.OK      # ~10 ms
    code = ctypes.c_int(-1)
    rc = lib.vqg_device_status(ctypes.byref(code))
    assert rc == _lib.ERR_DEVICE_TIMEOUT and code.value == 11
    assert V.device_status() == 0
    x, idx, cb = O.make_bl_inputs(4, 1024, 256, 4, 256, 128, seed=3)
    y = V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=128, layout="bl")
    torch.cuda.synchronize()
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, 128))


def test_rank_barrier_arguments_are_checked_on_the_host():
    lib = _lib.load()
    flags, arr = _flag_arrays(2)
    assert lib.vqg_rank_barrier(arr, 2, 2, 1, 20_000_000, None) == _lib.ERR_BAD_ARG      # rank out of range
    assert lib.vqg_rank_barrier(arr, 0, 9, 1, 20_000_000, None) == _lib.ERR_BAD_ARG      # too many ranks
    assert lib.vqg_rank_barrier(arr, 0, 2, 1, 10, None) == _lib.ERR_BAD_ARG              # limit too short
    assert lib.vqg_rank_barrier(arr, 0, 2, 1, 10**12, None) == _lib.ERR_BAD_ARG          # limit too long
    bad = (ctypes.c_void_p * 2)(flags[0].data_ptr(), None)
    assert lib.vqg_rank_barrier(bad, 0, 2, 1, 20_000_000, None) == _lib.ERR_BAD_ARG      # null flag array
