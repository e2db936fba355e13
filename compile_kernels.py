"""Build entry point, same command line as the reference's (compile_kernels.py:50-68):

    python compile_kernels.py build_ext --inplace

It builds ONE library for sm_100a, ``vq_gemm_b200/libvqg_b200.so`` (the C ABI of include/vqg.h,
compiled by nvcc without torch headers), and the PyTorch-extension shim ``vq_gemm_cuda.so`` at
the repository root (vq_gemm_b200/csrc/bind.cpp, compiled by g++ against torch and linked to the
C-ABI library).  There is no Triton, no backend dispatch and no CPU fallback.  The reference's
``KERNELS`` environment variable is accepted and ignored: all kernels live in the one library.
Pass ``--no-shim`` to build only the C-ABI library (seconds instead of a minute or two).
"""
import os
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def build_shim(force=False):
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    src = os.path.join(ROOT, "vq_gemm_b200", "csrc", "bind.cpp")
    out = os.path.join(ROOT, "vq_gemm_cuda.so")
    lib = os.path.join(ROOT, "vq_gemm_b200", "libvqg_b200.so")
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(lib)):
        return out
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           "-DTORCH_EXTENSION_NAME=vq_gemm_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    cmd += [src, "-o", out, f"-L{os.path.dirname(lib)}", "-lvqg_b200", "-Wl,-rpath,$ORIGIN/vq_gemm_b200"]
    for p in library_paths("cuda"):
        cmd += [f"-L{p}", f"-Wl,-rpath,{p}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    subprocess.run(cmd, check=True)
    return out


def main(argv):
    from vq_gemm_b200.build import build
    force = "--force" in argv
    print(build(force=force))
    if "--no-shim" not in argv:
        print(build_shim(force=force))


if __name__ == "__main__":
    main(sys.argv[1:])
