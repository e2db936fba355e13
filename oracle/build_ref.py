"""Recipe that compiles the reference's own CUDA kernels, unmodified and from where
they lie, into ``oracle/_ref/`` as PyTorch extension modules for sm_100a.

TEST / BASELINE INFRASTRUCTURE ONLY.  Nothing in the product package imports what
this builds; the GPU parity tests use it to pin the REF-layout path against the
reference's kernels and ``bench.py`` times it as a reported baseline.

It does not run the reference's build script (compile_kernels.py uses setuptools and
``-arch=sm_120a``); it issues one plain ``nvcc`` command per variant with the flags of
compile_kernels.py:6-17 re-targeted to ``-gencode arch=compute_100a,code=sm_100a``
(strategy_3 needs the explicit gencode form because of ``setmaxnreg``).

It also places an unmodified copy of the reference's harness (its ``bench.py``) in
``oracle/_ref/`` so that a GPU test can run that file itself against this build's modules on
a machine where the reference tree is not checked out (the copy is an output like the
``.so`` files: git-ignored, never committed).

Usage:  python oracle/build_ref.py [--ref /path/to/reference] [--only s1,s2_128] [-j 6]
        (the reference's location defaults to the environment variable VQG_REFERENCE_DIR)
Outputs ``oracle/_ref/vq_gemm_cuda_<variant>.so`` and ``oracle/_ref/bench.py``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# variant -> (source relative to the reference root, extra nvcc flags); compile_kernels.py:10-47
VARIANTS = {
    "cublas_gemm": ("ref_gemm/cublas_gemm_fp16.cu", ["-lcublas"]),
    "s1": ("strategy_1/src.cu", []),
    "s2_128": ("strategy_2/bsz128/src.cu", []),
    "s2_512": ("strategy_2/bsz512/src.cu", []),
    "s3_naive": ("strategy_3/naive/src.cu", ["--maxrregcount=128"]),
    "s3_wasp": ("strategy_3/wasp/src.cu", ["--maxrregcount=64", "-lcuda"]),
}


def _cmd(ref: str, variant: str) -> list[str]:
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    src, extra = VARIANTS[variant]
    name = f"vq_gemm_cuda_{variant}"
    inc = [f"-I{p}" for p in include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    lib = [f"-L{p}" for p in library_paths("cuda")]
    rpath = [f"-Xlinker=-rpath={p}" for p in library_paths("cuda")]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return (
        ["nvcc", "-shared", "-O2", "-lineinfo", "-std=c++17",
         "-gencode", "arch=compute_100a,code=sm_100a",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-O2", "-w",
         f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
         f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
         "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
         "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
         "--expt-relaxed-constexpr"]
        + inc + extra
        + [os.path.join(ref, "bind.cpp"), os.path.join(ref, src),
           "-o", os.path.join(OUT, name + ".so")]
        + lib + rpath
        + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    )


def build_one(ref: str, variant: str, force: bool) -> tuple[str, int, str]:
    src = os.path.join(ref, VARIANTS[variant][0])
    out = os.path.join(OUT, f"vq_gemm_cuda_{variant}.so")
    if (not force and os.path.exists(out)
            and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(os.path.join(ref, "bind.cpp")))):
        return variant, 0, "up to date"
    p = subprocess.run(_cmd(ref, variant), capture_output=True, text=True)
    return variant, p.returncode, (p.stdout + p.stderr)[-2000:]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("VQG_REFERENCE_DIR", ""))
    ap.add_argument("--only", default="")
    ap.add_argument("-j", type=int, default=6)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    if not a.ref or not os.path.isdir(a.ref):
        print(f"reference tree {a.ref!r} not present (set VQG_REFERENCE_DIR or pass --ref); nothing built")
        return 0
    os.makedirs(OUT, exist_ok=True)
    harness = os.path.join(a.ref, "bench.py")
    if os.path.exists(harness):
        shutil.copyfile(harness, os.path.join(OUT, "bench.py"))
    variants = [v for v in (a.only.split(",") if a.only else VARIANTS) if v]
    rc = 0
    with ThreadPoolExecutor(max_workers=a.j) as ex:
        for variant, code, log in ex.map(lambda v: build_one(a.ref, v, a.force), variants):
            print(f"[{variant}] rc={code} {log if code else log[-200:]}")
            rc |= code
    return rc


if __name__ == "__main__":
    sys.exit(main())
