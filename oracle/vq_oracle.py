"""CPU oracle for the vector-quantised GEMM hot path.

TEST INFRASTRUCTURE, NOT PRODUCT.  Only the tests, the smoke check and the CPU-baseline /
reference arms of the benchmark may import this module; the product package never does
and has no CPU path of its own.

It restates, in plain torch-on-CPU, what the reference's harness uses as ground truth:

* REF layout -- ``vq_gemm_reference`` in the reference's bench.py:37-57: indices
  ``w[K, Nq]`` (uint8), codebook ``[Nq/4, ENTRY, RATIO]``; the sub-vector of length RATIO
  runs along the OUTPUT dimension and 4 consecutive index columns share a codebook::

      Wdec[k, n*RATIO + r] = codebook[n // 4][ w[k, n] ][r]
      Y[M, Nq*RATIO]       = X[M, K] @ Wdec

  The reference multiplies with cuBLAS fp16 (ref_gemm/cublas_gemm_fp16.cu:36-46,
  CUBLAS_COMPUTE_16F, closed source, version unpinned).  This oracle accumulates in
  fp32 and rounds once to fp16, which is the contract the build is measured against.
  The gather half is pinned bit-exactly against the reference's own code by the
  fixtures in tests/golden (made by tests/golden/make_golden.py, which imports the
  reference's bench.py); the matmul half has no golden vector in the reference
  (bench.py:97-103 only prints differences): for it, parity is unpinned beyond the
  stated tolerance.

* BL layout -- the generalised format the benchmark configurations use; the reference
  has no implementation of it, so it is defined here by its scalar rule::

      W[n, v*j + r] = codebook[g(n)][ idx[n, j] ][r]     g(n) = n // rows_per_codebook
      Y[M, N]       = X[M, K] @ W^T                      (fp32 accumulate, fp16 out)

  ``idx`` is ``[N, K/v]`` uint8 (C <= 256) or uint16/int16 (C <= 65536, e.g. 12-bit values),
  ``codebook`` is ``[G, C, v]`` fp16 (``[C, v]`` = one codebook for the whole matrix).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

# Tolerance of the build contract: max|dY| / max|Yref| <= REL_TOL and, per element,
# |dY| <= ELT_TOL * (|Yref| + 1).
REL_TOL = 1e-2
ELT_TOL = 2e-2


def _as_index(idx: torch.Tensor) -> torch.Tensor:
    """Integer view of an index tensor as int64; uint16 stored in int16 is re-read unsigned."""
    if idx.dtype == torch.uint8:
        return idx.to(torch.int64)
    if idx.dtype == torch.int16:
        return idx.to(torch.int64) & 0xFFFF
    if idx.dtype == torch.uint16:
        return idx.view(torch.int16).to(torch.int64) & 0xFFFF
    if idx.dtype in (torch.int32, torch.int64):
        return idx.to(torch.int64)
    raise TypeError(f"unsupported index dtype {idx.dtype}")


def dequant_ref_layout(w: torch.Tensor, codebook: torch.Tensor) -> torch.Tensor:
    """REF-layout gather, following bench.py:41-55 of the reference.

    w [K, Nq] uint8, codebook [Nq/4, ENTRY, RATIO] fp16 -> Wdec [K, Nq*RATIO] fp16.
    """
    K, Nq = w.shape
    ratio = codebook.shape[2]
    group = torch.arange(Nq) // 4                       # bench.py:46
    group = group.unsqueeze(0).expand(K, Nq)            # bench.py:48
    entry = _as_index(w)                                # bench.py:50
    wdec = codebook[group, entry]                       # bench.py:53  [K, Nq, RATIO]
    return wdec.reshape(K, Nq * ratio).contiguous()     # bench.py:55


def dequant_bl_layout(idx: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int = 0) -> torch.Tensor:
    """BL-layout gather.  idx [N, K/v]; codebook [G, C, v] or [C, v] -> W [N, K] fp16."""
    if codebook.dim() == 2:
        codebook = codebook.unsqueeze(0)
    G, C, v = codebook.shape
    N, J = idx.shape
    if rows_per_codebook <= 0:
        rows_per_codebook = N if G == 1 else N // G
    group = (torch.arange(N) // rows_per_codebook).unsqueeze(1).expand(N, J)
    if group.numel() and int(group.max()) >= G:
        raise ValueError("not enough codebooks for N / rows_per_codebook")
    w = codebook[group, _as_index(idx)]                 # [N, J, v]
    return w.reshape(N, J * v).contiguous()


def dequant_bl_scalar(idx, codebook, rows_per_codebook: int = 0):
    """The BL rule as plain Python loops (small cases only); pins ``dequant_bl_layout``."""
    if codebook.dim() == 2:
        codebook = codebook.unsqueeze(0)
    G, C, v = codebook.shape
    N, J = idx.shape
    if rows_per_codebook <= 0:
        rows_per_codebook = N if G == 1 else N // G
    ii = _as_index(idx).tolist()
    out = torch.empty(N, J * v, dtype=codebook.dtype)
    for n in range(N):
        g = n // rows_per_codebook
        for j in range(J):
            for r in range(v):
                out[n, v * j + r] = codebook[g, ii[n][j], r]
    return out


def dequant_ref_scalar(w, codebook):
    """The REF rule as plain Python loops (small cases only)."""
    K, Nq = w.shape
    ratio = codebook.shape[2]
    ww = _as_index(w).tolist()
    out = torch.empty(K, Nq * ratio, dtype=codebook.dtype)
    for k in range(K):
        for n in range(Nq):
            for r in range(ratio):
                out[k, n * ratio + r] = codebook[n // 4, ww[k][n], r]
    return out


def dequant_bl_residual(idx: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int = 0) -> torch.Tensor:
    """Residual (multi-codebook) BL gather.  idx [S, N, K/v]; codebook [S, G, C, v] -> W [N, K] fp16 with

        W_0 = codebook_0[g(n)][idx_0[n, j]],   W_s = fp16(W_{s-1} + codebook_s[g(n)][idx_s[n, j]])

    i.e. the stages' entries added one after the other, every addition rounded to fp16 (round to nearest even;
    torch adds two fp16 tensors on the CPU by adding in fp32 and rounding, which is the same value).  The
    reference only names the idea (`#define RESIDUAL 1`, strategy_1/src.cu:18, never used), so the rule is
    this build's: parity unpinned against the reference."""
    S = idx.shape[0]
    w = dequant_bl_layout(idx[0], codebook[0], rows_per_codebook)
    for s in range(1, S):
        w = (w.float() + dequant_bl_layout(idx[s], codebook[s], rows_per_codebook).float()).half()
    return w


def dequant_bl_residual_scalar(idx, codebook, rows_per_codebook: int = 0):
    """The residual rule as plain Python loops over numpy float16 scalars (small cases only)."""
    import numpy as np
    S, N, J = idx.shape
    _, G, C, v = codebook.shape
    if rows_per_codebook <= 0:
        rows_per_codebook = N if G == 1 else N // G
    cbn = codebook.numpy()
    ii = [_as_index(idx[s]).tolist() for s in range(S)]
    out = np.empty((N, J * v), dtype=np.float16)
    for n in range(N):
        g = n // rows_per_codebook
        for j in range(J):
            for r in range(v):
                acc = cbn[0, g, ii[0][n][j], r]
                for s in range(1, S):
                    acc = np.float16(np.float32(acc) + np.float32(cbn[s, g, ii[s][n][j], r]))
                out[n, v * j + r] = acc
    return torch.from_numpy(out)


def vq_gemm_bl_residual(x, idx, codebook, rows_per_codebook: int = 0) -> torch.Tensor:
    return matmul_fp32acc(x, dequant_bl_residual(idx, codebook, rows_per_codebook))


def make_residual_inputs(M, K, N, v, C, rows_per_codebook=0, stages=2, seed=0, idx_dtype: Optional[torch.dtype] = None,
                         cb_sigma: float = 0.02):
    """Seeded inputs of the residual format: stage s has its own indices and codebooks, later stages smaller
    (sigma / 2^s) as a residual quantiser would leave them."""
    g = torch.Generator().manual_seed(seed)
    G = 1 if rows_per_codebook <= 0 else (N + rows_per_codebook - 1) // rows_per_codebook
    x = torch.randn(M, K, generator=g).half()
    cb = torch.stack([(torch.randn(G, C, v, generator=g) * (cb_sigma / 2 ** s)).half() for s in range(stages)])
    if idx_dtype is None:
        idx_dtype = torch.uint8 if C <= 256 else torch.int16
    idx = torch.randint(0, C, (stages, N, K // v), generator=g, dtype=torch.int32)
    idx = idx.to(torch.uint8) if idx_dtype == torch.uint8 else idx.to(torch.int16)
    return x, idx.contiguous(), cb.contiguous()


def matmul_fp32acc(x: torch.Tensor, w_nk: torch.Tensor) -> torch.Tensor:
    """Y = X @ W^T with fp32 accumulation and one rounding to fp16.  x [M,K], w_nk [N,K]."""
    return (x.float() @ w_nk.float().t()).half()


def vq_gemm_bl(x, idx, codebook, rows_per_codebook: int = 0) -> torch.Tensor:
    return matmul_fp32acc(x, dequant_bl_layout(idx, codebook, rows_per_codebook))


def vq_gemm_swiglu_bl(x, idx, codebook, rows_per_codebook: int = 0) -> torch.Tensor:
    """Gated product over (gate, up) row pairs (row 2i gate, row 2i+1 up): fp32 products, SiLU(g) * u in
    fp32, one rounding to fp16.  The reference has no such step; the rule is the one stated in
    include/vqg.h (the gather half is the pinned BL gather, the rest is torch fp32 arithmetic)."""
    w = dequant_bl_layout(idx, codebook, rows_per_codebook)
    p = x.float() @ w.float().t()
    g, u = p[:, 0::2], p[:, 1::2]
    return (g / (1.0 + torch.exp(-g)) * u).half()


def vq_gemm_ref_layout(x, w, codebook) -> torch.Tensor:
    wdec = dequant_ref_layout(w, codebook)              # [K, Nout]
    return (x.float() @ wdec.float()).half()


def vq_gemm_bl_rows(x, idx, codebook, rows_per_codebook: int, row_sel: torch.Tensor, col_sel: torch.Tensor):
    """Oracle on a subset: Y[row_sel][:, col_sel], for shapes whose full CPU result is too slow.

    Only the selected weight rows are dequantised; group membership uses the global row number.
    """
    if codebook.dim() == 2:
        codebook = codebook.unsqueeze(0)
    G = codebook.shape[0]
    N, J = idx.shape
    if rows_per_codebook <= 0:
        rows_per_codebook = N if G == 1 else N // G
    group = (col_sel // rows_per_codebook).unsqueeze(1).expand(col_sel.numel(), J)
    w = codebook[group, _as_index(idx[col_sel])].reshape(col_sel.numel(), -1)
    return (x[row_sel].float() @ w.float().t()).half()


def check_tolerance(y: torch.Tensor, y_ref: torch.Tensor, rel_tol: float = REL_TOL, elt_tol: float = ELT_TOL) -> dict:
    """Both bounds of the contract, with the statistics a reader wants to see."""
    y = y.detach().float().cpu()
    y_ref = y_ref.detach().float().cpu()
    if y.shape != y_ref.shape:
        return {"ok": False, "why": f"shape {tuple(y.shape)} != {tuple(y_ref.shape)}"}
    if y.numel() == 0:
        return {"ok": True, "max_abs": 0.0, "max_rel": 0.0, "n_bad": 0}
    d = (y - y_ref).abs()
    finite = bool(torch.isfinite(y).all())
    ref_max = float(y_ref.abs().max())
    max_abs = float(d.max())
    max_rel = max_abs / ref_max if ref_max > 0 else (0.0 if max_abs == 0 else math.inf)
    bad = d > elt_tol * (y_ref.abs() + 1.0)
    n_bad = int(bad.sum())
    return {
        "ok": finite and max_rel <= rel_tol and n_bad == 0,
        "finite": finite,
        "max_abs": max_abs,
        "mean_abs": float(d.mean()),
        "max_rel": max_rel,
        "max_elt_rel": float((d / y_ref.abs().clamp_min(1.0)).max()),
        "n_bad": n_bad,
        "ref_max": ref_max,
    }


def make_bl_inputs(M, K, N, v, C, rows_per_codebook=0, seed=0, idx_dtype: Optional[torch.dtype] = None,
                   cb_sigma: float = 0.02):
    """Seeded synthetic inputs with the value distributions of the benchmark configurations:
    X fp16 ~ N(0,1), codebook fp16 ~ N(0, cb_sigma), indices uniform in [0, C)."""
    g = torch.Generator().manual_seed(seed)
    G = 1 if rows_per_codebook <= 0 else (N + rows_per_codebook - 1) // rows_per_codebook
    x = torch.randn(M, K, generator=g).half()
    cb = (torch.randn(G, C, v, generator=g) * cb_sigma).half()
    if idx_dtype is None:
        idx_dtype = torch.uint8 if C <= 256 else torch.int16
    idx = torch.randint(0, C, (N, K // v), generator=g, dtype=torch.int32)
    idx = idx.to(torch.uint8) if idx_dtype == torch.uint8 else idx.to(torch.int16)
    return x, idx, cb


def make_ref_inputs(M, K, Nq, seed=42, entry=256, ratio=2):
    """Inputs shaped like the reference harness makes them (bench.py:83-85): randn X and
    codebook (sigma 1), uniform uint8 indices [K, Nq], codebook [Nq/4, ENTRY, RATIO]."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).half()
    w = torch.randint(0, entry, (K, Nq), generator=g, dtype=torch.int32).to(torch.uint8)
    cb = torch.randn(Nq // 4, entry, ratio, generator=g).half()
    return x, w, cb
