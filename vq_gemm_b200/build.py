"""Builds ``libvqg_b200.so`` (the C-ABI library, no torch headers) in-tree with nvcc for sm_100a.

    python -m vq_gemm_b200.build [--force] [--verbose]

One object per ``csrc/*.cu`` (compiled in parallel), linked with the static CUDA runtime so the
library loads on a machine without a GPU driver (the driver entry point for tensor-map
encoding is looked up at run time, not linked).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libvqg_b200.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime():
    ts = [os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC)]
    ts.append(os.path.getmtime(os.path.join(INCLUDE, "vqg.h")))
    return max(ts)


def _compile(src: str, verbose: bool):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    cmd = ["nvcc", *NVCC_FLAGS, f"-I{INCLUDE}", "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    p = subprocess.run(cmd, capture_output=True, text=True)
    return src, obj, p.returncode, p.stdout + p.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles if anything under csrc/ or include/ is newer than the library; returns its path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    objs = []
    with ThreadPoolExecutor(max_workers=8) as ex:
        for src, obj, rc, log in ex.map(lambda s: _compile(s, verbose), _sources()):
            if verbose or rc:
                sys.stderr.write(f"--- {src}\n{log}\n")
            if rc:
                raise RuntimeError(f"nvcc failed on {src}")
            objs.append(obj)
    link = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs,
            "-cudart", "static", "-Xcompiler", "-fPIC"]
    p = subprocess.run(link, capture_output=True, text=True)
    if p.returncode:
        raise RuntimeError("link failed:\n" + p.stdout + p.stderr)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
