"""Quantiser and packer: dense fp16 weights -> (indices, codebooks) of the generalised format.

The step before the product.  The reference has none (its benchmark fills ``w`` with random bytes,
bench.py:83-85), so the rules are this library's own and are written down where they are exact:

* ``assign``: nearest codebook entry per length-``v`` sub-vector under the squared Euclidean
  distance, summed in fp32 in index order with every operation rounded separately, lowest index on
  ties (``vqg_quantize_assign``).
* ``kmeans_update``: one Lloyd step with exact, order-independent sums (``vqg_quantize_update``).
* ``kmeans_quantize``: seeded initialisation from the data + ``iters`` x (assign, update) + assign.
* ``pack12`` / ``unpack12``: 12-bit storage for indices into 4096-entry codebooks.

Everything runs on the GPU through the C ABI; there is no CPU path here.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .ops import _idx_bytes, _require_cuda, _stream_ptr


def _shape(weight: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int):
    if weight.dim() != 2 or weight.dtype != torch.float16:
        raise RuntimeError("weight must be a float16 [N, K] tensor")
    cb3 = codebook if codebook.dim() == 3 else codebook.unsqueeze(0)
    if cb3.dtype != torch.float16:
        raise RuntimeError("codebook must be float16")
    N, K = weight.shape
    G, C, v = cb3.shape
    if K % v:
        raise RuntimeError("K must be a multiple of v")
    groups = 1 if (rows_per_codebook <= 0 or rows_per_codebook >= N) else -(-N // rows_per_codebook)
    if G < groups:
        raise RuntimeError(f"{G} codebooks given, {groups} needed")
    return N, K, C, v


def assign(weight: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int = 0,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Indices [N, K/v] of the nearest entries (uint8 for up to 256 entries, int16 above)."""
    lib = _lib.load()
    dev = _require_cuda(weight, codebook)
    N, K, C, v = _shape(weight, codebook, rows_per_codebook)
    dtype = torch.uint8 if C <= 256 else torch.int16
    if out is None:
        out = torch.empty((N, K // v), dtype=dtype, device=dev)
    elif tuple(out.shape) != (N, K // v) or not out.is_contiguous() or out.device != dev:
        raise RuntimeError("out must be a contiguous [N, K/v] index tensor on the inputs' device")
    with torch.cuda.device(dev):
        st = lib.vqg_quantize_assign(weight.data_ptr(), codebook.data_ptr(), out.data_ptr(), N, K, v, C, _idx_bytes(out),
                                     rows_per_codebook, _stream_ptr(dev))
    _lib.check(st, "quantize.assign")
    return out


def kmeans_update(weight: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int = 0) -> torch.Tensor:
    """One Lloyd update of ``codebook`` in place (returns it)."""
    lib = _lib.load()
    dev = _require_cuda(weight, indices, codebook)
    N, K, C, v = _shape(weight, codebook, rows_per_codebook)
    if tuple(indices.shape) != (N, K // v):
        raise RuntimeError("indices must be [N, K/v]")
    with torch.cuda.device(dev):
        nbytes = lib.vqg_quantize_workspace_bytes(N, v, C, rows_per_codebook)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        st = lib.vqg_quantize_update(weight.data_ptr(), indices.data_ptr(), codebook.data_ptr(), ws.data_ptr(), nbytes, N, K,
                                     v, C, _idx_bytes(indices), rows_per_codebook, _stream_ptr(dev))
    _lib.check(st, "quantize.kmeans_update")
    return codebook


def initial_codebook(weight: torch.Tensor, v: int, entries: int, rows_per_codebook: int = 0, seed: int = 0) -> torch.Tensor:
    """[G, entries, v]: for every group, ``entries`` sub-vectors of the group drawn with a seeded CPU
    generator (positions ``randint(0, sub-vectors of the group)``; repeats allowed)."""
    N, K = weight.shape
    rpc = N if (rows_per_codebook <= 0 or rows_per_codebook >= N) else rows_per_codebook
    G = -(-N // rpc)
    J = K // v
    gen = torch.Generator().manual_seed(seed)
    subs = weight.reshape(N * J, v)
    picks = []
    for g in range(G):
        rows = min(rpc, N - g * rpc)
        pos = torch.randint(0, rows * J, (entries,), generator=gen) + g * rpc * J
        picks.append(pos)
    pos = torch.stack(picks).to(weight.device)
    return subs[pos.reshape(-1)].reshape(G, entries, v).contiguous()


def kmeans_quantize(weight: torch.Tensor, *, v: int = 8, entries: int = 256, rows_per_codebook: int = 128, iters: int = 10,
                    seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(indices [N, K/v], codebook [G, entries, v]) for a float16 CUDA weight [N, K]."""
    weight = weight.contiguous()
    cb = initial_codebook(weight, v, entries, rows_per_codebook, seed)
    idx = assign(weight, cb, rows_per_codebook)
    for _ in range(iters):
        kmeans_update(weight, idx, cb, rows_per_codebook)
        assign(weight, cb, rows_per_codebook, out=idx)
    # The small-batch product kernels read their weights before they wait for the kernel ahead of them on the
    # stream (programmatic dependent launch).  The library orders its own quantiser kernels against the next
    # product on the same stream, so the returned tensors can be used at once on this stream.
    return idx, cb


def kmeans_quantize_residual(weight: torch.Tensor, *, stages: int = 2, v: int = 8, entries: int = 256,
                             rows_per_codebook: int = 128, iters: int = 10, seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Residual (multi-codebook) quantisation: stage 0 quantises the weight, every further stage quantises what the
    stages before it left over, so that ``W ~ fp16(... fp16(cb_0[idx_0] + cb_1[idx_1]) ...)`` -- the running fp16 sum
    the residual format is defined by.  Returns (indices [S, N, K/v], codebook [S, G, entries, v])."""
    from .ops import dequant_residual
    if stages < 1 or stages > 8:
        raise RuntimeError("stages must be between 1 and 8")
    weight = weight.contiguous()
    idx_all = cb_all = None
    target = weight
    for s in range(stages):
        idx, cb = kmeans_quantize(target, v=v, entries=entries, rows_per_codebook=rows_per_codebook, iters=iters, seed=seed + s)
        if idx_all is None:
            idx_all = torch.empty((stages,) + tuple(idx.shape), dtype=idx.dtype, device=idx.device)
            cb_all = torch.empty((stages,) + tuple(cb.shape), dtype=cb.dtype, device=cb.device)
        # contiguous same-type device copies are plain stream-ordered memory copies, which the product kernels'
        # early weight reads are ordered against (unlike a kernel's writes)
        idx_all[s].copy_(idx)
        cb_all[s].copy_(cb)
        if s + 1 < stages:
            so_far = dequant_residual(idx_all[:s + 1], cb_all[:s + 1], rows_per_codebook=rows_per_codebook)
            target = (weight.float() - so_far.float()).half()
    return idx_all, cb_all


def pack12(indices: torch.Tensor) -> torch.Tensor:
    """int16/uint16 indices < 4096, even count per row -> uint8 [..., 3/2 * last]."""
    lib = _lib.load()
    dev = _require_cuda(indices)
    if indices.dtype not in (torch.int16, torch.uint16) or indices.shape[-1] % 2:
        raise RuntimeError("pack12 expects (u)int16 indices with an even last dimension")
    out = torch.empty((*indices.shape[:-1], indices.shape[-1] * 3 // 2), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        st = lib.vqg_pack12(indices.data_ptr(), out.data_ptr(), indices.numel(), _stream_ptr(dev))
    _lib.check(st, "pack12")
    return out


def unpack12(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack12`: uint8 [..., 3m] -> int16 [..., 2m]."""
    lib = _lib.load()
    dev = _require_cuda(packed)
    if packed.dtype != torch.uint8 or packed.shape[-1] % 3:
        raise RuntimeError("unpack12 expects uint8 with a last dimension that is a multiple of 3")
    out = torch.empty((*packed.shape[:-1], packed.shape[-1] * 2 // 3), dtype=torch.int16, device=dev)
    with torch.cuda.device(dev):
        st = lib.vqg_unpack12(packed.data_ptr(), out.data_ptr(), out.numel(), _stream_ptr(dev))
    _lib.check(st, "unpack12")
    return out
