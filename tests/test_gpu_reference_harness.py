"""Runs the reference's own harness file, unmodified, against this build's extension modules.

oracle/build_ref.py places a byte-for-byte copy of the reference's ``bench.py`` in ``oracle/_ref/``
(an output, never committed).  Here that file is started as a child process the way the reference's
Makefile does it (``KERNELS=<variant> python bench.py``, Makefile:20-21) with ``compat/`` on the module
path, so that its six unconditional imports (bench.py:6-11) resolve to the single sm_100a extension
and its ``matplotlib`` import to the numeric stand-in.  What the harness prints is checked: the shape
line, the error statistics against its own torch-gather + ``gemm`` oracle (bench.py:92-103) and the
four "run 0 vs i" determinism lines for the kernel and for the oracle (bench.py:118-132).

The harness draws codebooks with sigma 1, so outputs have sigma 64 and lie below 512: the kernel and
the harness's oracle (this build's dense product) both accumulate in fp32 and round once to fp16,
hence they may differ by one fp16 step of the largest outputs (0.25) and no more.
"""
import os
import re
import subprocess
import sys

import pytest

from tests._util import ROOT

pytestmark = pytest.mark.gpu

HARNESS = os.path.join(ROOT, "oracle", "_ref", "bench.py")


def _run(tmp_path, **env_extra):
    if not os.path.exists(HARNESS):
        pytest.skip("oracle/_ref/bench.py not present (python oracle/build_ref.py copies it from a reference checkout)")
    if not os.path.exists(os.path.join(ROOT, "vq_gemm_cuda.so")):
        pytest.fail("vq_gemm_cuda.so is missing: run `python compile_kernels.py build_ext --inplace`")
    (tmp_path / "figures").mkdir()
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(ROOT, "compat"), ROOT, env.get("PYTHONPATH", "")])
    env["PYTHONIOENCODING"] = "utf-8"
    env.update(env_extra)
    p = subprocess.run([sys.executable, HARNESS], cwd=tmp_path, env=env, capture_output=True, text=True, timeout=600,
                       encoding="utf-8")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    return p.stdout


@pytest.mark.parametrize("variant", ["s3_wasp", "s1"])
def test_reference_harness_runs_unchanged(tmp_path, variant):
    out = _run(tmp_path, KERNELS=variant)
    assert f"Using kernel VERSION={variant}" in out
    assert "M=2048, K=4096, N=640, ENTRY=256, RATIO=2" in out                 # bench.py:13-15,29-30
    assert "VQ GEMM output shape:torch.Size([2048, 1280])" in out
    mean = float(re.search(r"Mean absolute difference \(CUDA vs Reference\): ([0-9.eE+-]+)", out).group(1))
    mx = float(re.search(r"Max abs diff: ([0-9.eE+-]+)", out).group(1))
    assert mean <= 0.02 and mx <= 0.25, (mean, mx)
    for i in range(1, 5):                                                     # bench.py:124-132
        assert f"CUDA output run 0 vs {i}: 一致" in out
        assert f"Reference output run 0 vs {i}: 一致" in out
    assert "不一致" not in out
    assert (tmp_path / "figures" / "M=2048_N=640_K=4096_err.npy").exists()    # the heat map, as numbers


def test_reference_harness_plain_gemm_mode(tmp_path):
    out = _run(tmp_path, KERNELS="s1", TEST_GEMM="TRUE")                      # Makefile:59 (run-gemm-128)
    assert "------------ test gemm ------------" in out
    mx = float(re.search(r"Max abs diff: ([0-9.eE+-]+)", out).group(1))
    assert mx == 0.0                                                          # both sides are the same dense kernel
