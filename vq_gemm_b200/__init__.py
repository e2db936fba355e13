"""B200 (sm_100a) vector-quantised GEMM: Y[M,N] = X[M,K] @ dequant(idx, codebook)^T.

The package is a thin host layer over ``libvqg_b200.so`` (C ABI in include/vqg.h).  It mirrors
the reference extension's entry points -- ``e2e_gemm`` and ``gemm`` -- and adds ``vq_gemm`` and
``dequant`` for the generalised weight format.  There is no CPU implementation.
"""
from .formats import CONFIGS, VQShape, infer_layout, make_inputs  # noqa: F401
from . import quantize  # noqa: F401
from .ops import (auto_path, dequant, dequant_residual, device_status, e2e_gemm, gemm, interleave_gate_up, launch_count,  # noqa: F401
                  vq_gemm, vq_gemm_residual, vq_gemm_swiglu)

__all__ = ["e2e_gemm", "gemm", "vq_gemm", "vq_gemm_swiglu", "vq_gemm_residual", "interleave_gate_up", "dequant",
           "dequant_residual", "auto_path", "quantize", "device_status", "launch_count", "CONFIGS", "VQShape", "infer_layout", "make_inputs"]
