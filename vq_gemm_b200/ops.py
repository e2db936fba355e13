"""Host-side mirror of the reference's extension module (bind.cpp:3-8) on top of the C ABI.

    e2e_gemm(input, w, codebook) -> o      same positional signature as the reference
    gemm(input, w) -> o                    dense fp16 product, w given as [K, N]
    vq_gemm(x, indices, codebook, ...)     generalised entry point (both weight formats)
    vq_gemm_swiglu(x, indices, codebook)   gated product SiLU(X g) * (X u) over (gate, up) row pairs
    vq_gemm_residual(x, indices, codebook) residual (multi-codebook) weights: indices [S, N, K/v], codebook [S, G, C, v]
    dequant(indices, codebook, ...)        bit-exact dequantised weights

All tensors must be CUDA tensors on one device; the output is allocated by the callee on that
device (the reference hard-codes device 0, strategy_1/src.cu:343) and the launch goes to torch's
current stream (the reference uses the legacy default stream).  Errors raise ``RuntimeError``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from .formats import infer_layout

_workspaces: dict = {}
_retired: list = []          # outgrown workspaces, kept alive (see _ws)
_MIN_WORKSPACE = 64 << 20    # covers the prefill kernel's partial tiles (37 MiB) and typical split-K partials


def _ws(device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Cached, zero-initialised scratch per (device, stream).  The library keeps the counter region zero
    between calls.  A workspace that has to grow is replaced by a larger one but never freed: a CUDA graph
    captured earlier may still hold its address, and memory handed back to the allocator could be given
    to another tensor of the same graph."""
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    cur = _workspaces.get(key)
    if cur is None or cur.numel() < nbytes:
        if cur is not None:
            _retired.append(cur)
        size = max(nbytes, _MIN_WORKSPACE, 2 * cur.numel() if cur is not None else 0)
        cur = torch.zeros(size, dtype=torch.uint8, device=device)
        _workspaces[key] = cur
    return cur


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("vq_gemm_b200 has no CPU path: all tensors must be CUDA tensors")
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same CUDA device")
        if not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous")
    return dev


def _idx_bytes(indices: torch.Tensor) -> int:
    if indices.dtype == torch.uint8:
        return 1
    if indices.dtype in (torch.int16, torch.uint16):
        return 2
    raise RuntimeError(f"indices must be uint8 or (u)int16, got {indices.dtype}")


def _stream_ptr(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def auto_path(M: int, N: int, K: int, v: int, C: int, index_bits: int = 8, rows_per_codebook: int = 0, layout: str = "bl") -> str:
    """Name of the kernel route the library picks by itself for a problem (``vqg_auto_path``)."""
    ib = {8: 1, 16: 2, 12: _lib.IDX_PACKED12}[index_bits]
    code = _lib.load().vqg_auto_path(M, N, K, v, C, ib, rows_per_codebook, _lib.LAYOUT_BL if layout == "bl" else _lib.LAYOUT_REF)
    return {val: name for name, val in _lib.PATHS.items()}.get(code, str(code))


def _packed12(indices: torch.Tensor, index_bits: Optional[int]) -> bool:
    if index_bits in (None, 8, 16):
        return False
    if index_bits != 12:
        raise RuntimeError("index_bits must be 8, 16 or 12 (packed)")
    if indices.dtype != torch.uint8 or indices.dim() != 2 or indices.shape[1] % 3:
        raise RuntimeError("packed 12-bit indices are a uint8 [N, K/v * 3/2] tensor (quantize.pack12)")
    return True


def vq_gemm(x: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor, *, rows_per_codebook: Optional[int] = None,
            layout: str = "auto", path: str = "auto", out: Optional[torch.Tensor] = None,
            index_bits: Optional[int] = None) -> torch.Tensor:
    """Y = X @ dequant(indices, codebook)^T, fp16 in and out, fp32 accumulation.
    ``index_bits=12``: `indices` holds 12-bit indices packed two to three bytes (``quantize.pack12``)."""
    lib = _lib.load()
    dev = _require_cuda(x, indices, codebook)
    if x.dtype != torch.float16 or codebook.dtype != torch.float16:
        raise RuntimeError("x and codebook must be float16")
    packed = _packed12(indices, index_bits)
    if layout == "auto":
        layout = "bl" if packed else infer_layout(x, indices, codebook)
    M, K = x.shape
    ib = _lib.IDX_PACKED12 if packed else _idx_bytes(indices)
    if packed and layout != "bl":
        raise RuntimeError("packed indices exist in the generalised format only")
    if layout == "bl":
        N = indices.shape[0]
        cb3 = codebook if codebook.dim() == 3 else codebook.unsqueeze(0)
        G, C, v = cb3.shape
        J = indices.shape[1] * 2 // 3 if packed else indices.shape[1]
        if J * v != K:
            raise RuntimeError(f"indices [N, K/v] = {tuple(indices.shape)} does not match K={K}, v={v}")
        if rows_per_codebook is None:
            if G == 1:
                rows_per_codebook = 0
            elif N % G == 0:
                rows_per_codebook = N // G
            else:
                raise RuntimeError("cannot infer rows_per_codebook: N is not a multiple of the number of codebooks")
        need_groups = 1 if rows_per_codebook <= 0 else -(-N // rows_per_codebook)
        if G < need_groups:
            raise RuntimeError(f"{G} codebooks given, {need_groups} needed")
        lay = _lib.LAYOUT_BL
    elif layout == "ref":
        Kw, Nq = indices.shape
        if Kw != K or codebook.dim() != 3 or tuple(codebook.shape) != (Nq // 4, 256, 2) or Nq % 4 or ib != 1:
            raise RuntimeError("reference format needs w [K, Nq] uint8 and codebook [Nq/4, 256, 2]")
        N, v, C, rows_per_codebook = 2 * Nq, 2, 256, 0
        lay = _lib.LAYOUT_REF
    else:
        raise RuntimeError(f"unknown layout {layout!r}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
    elif tuple(out.shape) != (M, N) or out.dtype != torch.float16 or not out.is_contiguous() or out.device != dev:
        raise RuntimeError("out must be a contiguous float16 [M, N] tensor on the inputs' device")
    pth = _lib.PATHS[path]
    with torch.cuda.device(dev):
        nbytes = lib.vqg_workspace_bytes(M, N, K, v, C, ib, rows_per_codebook, lay, pth)
        ws = _ws(dev, nbytes)
        st = lib.vqg_gemm_path(x.data_ptr(), indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), M, N, K, v, C, ib,
                               rows_per_codebook, lay, pth, ws.data_ptr() if ws is not None else None,
                               ws.numel() if ws is not None else 0, _stream_ptr(dev))
    _lib.check(st, "vq_gemm")
    return out


def _residual_dims(indices: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: Optional[int]):
    if indices.dim() != 3 or codebook.dim() != 4 or indices.shape[0] != codebook.shape[0]:
        raise RuntimeError("residual weights need indices [S, N, K/v] and codebook [S, G, C, v] with the same S")
    S, N, J = indices.shape
    _, G, C, v = codebook.shape
    if rows_per_codebook is None:
        rows_per_codebook = 0 if G == 1 else N // G
    need_groups = 1 if rows_per_codebook <= 0 else -(-N // rows_per_codebook)
    if G != need_groups:
        raise RuntimeError(f"{G} codebooks per stage given, {need_groups} needed (stages are stored back to back)")
    return S, N, J, G, C, v, rows_per_codebook


def vq_gemm_residual(x: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor, *,
                     rows_per_codebook: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y = X @ W^T for residual (multi-codebook) weights: indices [S, N, K/v], codebook [S, G, C, v],
    W = the running fp16 sum over the stages of the looked-up entries (see include/vqg.h)."""
    lib = _lib.load()
    dev = _require_cuda(x, indices, codebook)
    if x.dtype != torch.float16 or codebook.dtype != torch.float16:
        raise RuntimeError("x and codebook must be float16")
    S, N, J, G, C, v, rpc = _residual_dims(indices, codebook, rows_per_codebook)
    M, K = x.shape
    if J * v != K:
        raise RuntimeError(f"indices [S, N, K/v] = {tuple(indices.shape)} do not match K={K}, v={v}")
    ib = _idx_bytes(indices)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
    elif tuple(out.shape) != (M, N) or out.dtype != torch.float16 or not out.is_contiguous() or out.device != dev:
        raise RuntimeError("out must be a contiguous float16 [M, N] tensor on the inputs' device")
    with torch.cuda.device(dev):
        ws = _ws(dev, lib.vqg_residual_workspace_bytes(M, N, K, v, C, ib, rpc, S))
        st = lib.vqg_gemm_residual(x.data_ptr(), indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), M, N, K, v, C, ib,
                                   rpc, S, ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                   _stream_ptr(dev))
    _lib.check(st, "vq_gemm_residual")
    return out


def _weights_out(out: Optional[torch.Tensor], shape, dev) -> torch.Tensor:
    if out is None:
        return torch.empty(shape, dtype=torch.float16, device=dev)
    if tuple(out.shape) != tuple(shape) or out.dtype != torch.float16 or out.device != dev or not out.is_contiguous():
        raise RuntimeError(f"out must be a contiguous float16 tensor of shape {tuple(shape)} on {dev}")
    return out


def dequant_residual(indices: torch.Tensor, codebook: torch.Tensor, *, rows_per_codebook: Optional[int] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dequantised residual weights [N, K], bit-exact by the format's rule."""
    lib = _lib.load()
    dev = _require_cuda(indices, codebook)
    if codebook.dtype != torch.float16:
        raise RuntimeError("codebook must be float16")
    S, N, J, G, C, v, rpc = _residual_dims(indices, codebook, rows_per_codebook)
    out = _weights_out(out, (N, J * v), dev)
    with torch.cuda.device(dev):
        st = lib.vqg_dequant_residual(indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), N, J * v, v, C,
                                      _idx_bytes(indices), rpc, S, _stream_ptr(dev))
    _lib.check(st, "dequant_residual")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Row-interleaves two [N, ...] tensors (dense weights or index matrices) into the [2N, ...] order
    the gated product expects: row 2i = gate row i, row 2i+1 = up row i."""
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise RuntimeError("gate and up must have the same shape and dtype")
    return torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], *gate.shape[1:]).contiguous()


def vq_gemm_swiglu(x: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor, *,
                   rows_per_codebook: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y[M, N/2] = SiLU(X g_i^T) * (X u_i^T) for a BL-format weight whose rows are (gate, up) pairs
    (see :func:`interleave_gate_up`); fp32 accumulation and combination, one rounding to fp16."""
    lib = _lib.load()
    dev = _require_cuda(x, indices, codebook)
    if x.dtype != torch.float16 or codebook.dtype != torch.float16:
        raise RuntimeError("x and codebook must be float16")
    M, K = x.shape
    ib = _idx_bytes(indices)
    N = indices.shape[0]
    if N % 2:
        raise RuntimeError("the gated product needs an even number of weight rows (gate, up pairs)")
    cb3 = codebook if codebook.dim() == 3 else codebook.unsqueeze(0)
    G, C, v = cb3.shape
    if indices.dim() != 2 or indices.shape[1] * v != K:
        raise RuntimeError(f"indices [N, K/v] = {tuple(indices.shape)} does not match K={K}, v={v}")
    if rows_per_codebook is None:
        rows_per_codebook = 0 if G == 1 else N // G
    need_groups = 1 if rows_per_codebook <= 0 else -(-N // rows_per_codebook)
    if G < need_groups:
        raise RuntimeError(f"{G} codebooks given, {need_groups} needed")
    n_out = N // 2
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.float16, device=dev)
    elif tuple(out.shape) != (M, n_out) or out.dtype != torch.float16 or not out.is_contiguous() or out.device != dev:
        raise RuntimeError("out must be a contiguous float16 [M, N/2] tensor on the inputs' device")
    with torch.cuda.device(dev):
        nbytes = lib.vqg_swiglu_workspace_bytes(M, n_out, K, v, C, ib, rows_per_codebook)
        ws = _ws(dev, nbytes)
        st = lib.vqg_gemm_swiglu(x.data_ptr(), indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), M, n_out, K, v, C, ib,
                                 rows_per_codebook, ws.data_ptr() if ws is not None else None,
                                 ws.numel() if ws is not None else 0, _stream_ptr(dev))
    _lib.check(st, "vq_gemm_swiglu")
    return out


def e2e_gemm(input: torch.Tensor, w: torch.Tensor, codebook: torch.Tensor) -> torch.Tensor:
    """Drop-in for the reference's ``e2e_gemm`` (bind.cpp:3,7).  Accepts the reference's format
    (w [K, Nq] uint8, codebook [Nq/4, 256, 2]) and, by shape, the generalised one."""
    return vq_gemm(input, w, codebook)


def gemm(input: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Drop-in for the reference's ``gemm`` (bind.cpp:4,8): input [M, K] @ w [K, N], fp16."""
    lib = _lib.load()
    dev = _require_cuda(input, w)
    if input.dtype != torch.float16 or w.dtype != torch.float16:
        raise RuntimeError("gemm expects float16 tensors")
    M, K = input.shape
    if w.dim() != 2 or w.shape[0] != K:
        raise RuntimeError("gemm expects w [K, N]")
    N = w.shape[1]
    out = torch.empty((M, N), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        ws = _ws(dev, lib.vqg_dense_workspace_bytes(M, N, K, 1))
        st = lib.vqg_dense_gemm(input.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, 1,
                                ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                _stream_ptr(dev))
    _lib.check(st, "gemm")
    return out


def dequant(indices: torch.Tensor, codebook: torch.Tensor, *, rows_per_codebook: Optional[int] = None,
            layout: str = "bl", out: Optional[torch.Tensor] = None, index_bits: Optional[int] = None) -> torch.Tensor:
    """Dequantised weights: ``[N, K]`` for the generalised format, ``[K, 2*Nq]`` for the reference's.
    ``index_bits=12``: packed indices as in :func:`vq_gemm`."""
    lib = _lib.load()
    dev = _require_cuda(indices, codebook)
    if codebook.dtype != torch.float16:
        raise RuntimeError("codebook must be float16")
    packed = _packed12(indices, index_bits)
    ib = _lib.IDX_PACKED12 if packed else _idx_bytes(indices)
    if packed and layout != "bl":
        raise RuntimeError("packed indices exist in the generalised format only")
    if layout == "bl":
        cb3 = codebook if codebook.dim() == 3 else codebook.unsqueeze(0)
        G, C, v = cb3.shape
        N, J = indices.shape
        if packed:
            J = J * 2 // 3
        K = J * v
        if rows_per_codebook is None:
            rows_per_codebook = 0 if G == 1 else N // G
        out = _weights_out(out, (N, K), dev)
        args = (N, K, v, C, ib, rows_per_codebook, _lib.LAYOUT_BL)
    elif layout == "ref":
        K, Nq = indices.shape
        out = _weights_out(out, (K, 2 * Nq), dev)
        args = (2 * Nq, K, 2, 256, ib, 0, _lib.LAYOUT_REF)
    else:
        raise RuntimeError(f"unknown layout {layout!r}")
    with torch.cuda.device(dev):
        st = lib.vqg_dequant(indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), *args, _stream_ptr(dev))
    _lib.check(st, "dequant")
    return out


def device_status() -> int:
    """Reads and clears the device status word (0 = no bounded wait has run out)."""
    code = ctypes.c_int(0)
    _lib.load().vqg_device_status(ctypes.byref(code))
    return code.value


def launch_count() -> int:
    return int(_lib.load().vqg_launch_count())
