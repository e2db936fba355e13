"""Alias of the single sm_100a extension under one of the reference's six module names
(reference compile_kernels.py:57-60; bench.py:6-11 imports all of them unconditionally)."""
from vq_gemm_cuda import dequant, e2e_gemm, gemm, vq_gemm  # noqa: F401
