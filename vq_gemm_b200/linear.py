"""Caller side of the boundary: the VQ-GEMM as a registered torch operator and an ``nn.Module``.

The reference stops at ``bench.py`` calling ``e2e_gemm`` on raw tensors (bench.py:66-80); a model
needs the product as a layer.  ``vq_gemm_b200::vq_linear`` is registered with ``torch.library`` so
that it can be traced (a fake-tensor rule gives shapes and dtypes without running anything), used
under ``torch.compile`` as an opaque call, and captured in CUDA graphs: the launch allocates nothing
but its output, and the scratch it uses is cached per (device, stream) and left as it found it.

Inference only: no autograd formula is registered.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import ops


@torch.library.custom_op("vq_gemm_b200::vq_linear", mutates_args=(), device_types="cuda")
def vq_linear(x: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int) -> torch.Tensor:
    """x [M, K] fp16, indices [N, K/v] uint8/int16, codebook [G, C, v] fp16 -> [M, N] fp16."""
    return ops.vq_gemm(x, indices, codebook, rows_per_codebook=rows_per_codebook, layout="bl")


@vq_linear.register_fake
def _(x, indices, codebook, rows_per_codebook):
    if x.dim() != 2 or indices.dim() != 2 or codebook.dim() != 3:
        raise RuntimeError("vq_linear expects x [M, K], indices [N, K/v], codebook [G, C, v]")
    if indices.shape[1] * codebook.shape[2] != x.shape[1]:
        raise RuntimeError("indices [N, K/v] and codebook [G, C, v] do not match x [M, K]")
    return x.new_empty((x.shape[0], indices.shape[0]))


@torch.library.custom_op("vq_gemm_b200::vq_linear_residual", mutates_args=(), device_types="cuda")
def vq_linear_residual(x: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int) -> torch.Tensor:
    """Residual weights: x [M, K] fp16, indices [S, N, K/v], codebook [S, G, C, v] fp16 -> [M, N] fp16."""
    return ops.vq_gemm_residual(x, indices, codebook, rows_per_codebook=rows_per_codebook)


@vq_linear_residual.register_fake
def _(x, indices, codebook, rows_per_codebook):
    if x.dim() != 2 or indices.dim() != 3 or codebook.dim() != 4 or indices.shape[0] != codebook.shape[0]:
        raise RuntimeError("vq_linear_residual expects x [M, K], indices [S, N, K/v], codebook [S, G, C, v]")
    if indices.shape[2] * codebook.shape[3] != x.shape[1]:
        raise RuntimeError("indices [S, N, K/v] and codebook [S, G, C, v] do not match x [M, K]")
    return x.new_empty((x.shape[0], indices.shape[1]))


@torch.library.custom_op("vq_gemm_b200::vq_linear_packed12", mutates_args=(), device_types="cuda")
def vq_linear_packed12(x: torch.Tensor, packed: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int) -> torch.Tensor:
    """12-bit indices packed two to three bytes: x [M, K] fp16, packed [N, K/v * 3/2] uint8, codebook [G, C, v]."""
    return ops.vq_gemm(x, packed, codebook, rows_per_codebook=rows_per_codebook, layout="bl", index_bits=12)


@vq_linear_packed12.register_fake
def _(x, packed, codebook, rows_per_codebook):
    if x.dim() != 2 or packed.dim() != 2 or codebook.dim() != 3 or packed.shape[1] % 3:
        raise RuntimeError("vq_linear_packed12 expects x [M, K], packed [N, K/v * 3/2], codebook [G, C, v]")
    if packed.shape[1] * 2 // 3 * codebook.shape[2] != x.shape[1]:
        raise RuntimeError("packed [N, K/v * 3/2] and codebook [G, C, v] do not match x [M, K]")
    return x.new_empty((x.shape[0], packed.shape[0]))


@torch.library.custom_op("vq_gemm_b200::vq_swiglu", mutates_args=(), device_types="cuda")
def vq_swiglu(x: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int) -> torch.Tensor:
    """x [M, K]; indices [2*N_out, K/v] with (gate, up) row pairs -> SiLU(x g^T) * (x u^T), [M, N_out] fp16."""
    return ops.vq_gemm_swiglu(x, indices, codebook, rows_per_codebook=rows_per_codebook)


@vq_swiglu.register_fake
def _(x, indices, codebook, rows_per_codebook):
    if x.dim() != 2 or indices.dim() != 2 or codebook.dim() != 3 or indices.shape[0] % 2:
        raise RuntimeError("vq_swiglu expects x [M, K], indices [2*N_out, K/v], codebook [G, C, v]")
    if indices.shape[1] * codebook.shape[2] != x.shape[1]:
        raise RuntimeError("indices [2*N_out, K/v] and codebook [G, C, v] do not match x [M, K]")
    return x.new_empty((x.shape[0], indices.shape[0] // 2))


class VQLinear(nn.Module):
    """``y = x @ dequant(indices, codebook)^T (+ bias)`` with the weight kept in compressed form.

    ``indices`` [out_features, in_features / v] (uint8, or int16 for codebooks of more than 256
    entries), ``codebook`` [groups, C, v] fp16 with one codebook per ``rows_per_codebook``
    consecutive output features (0: a single codebook).  Both are buffers, so ``state_dict`` /
    ``load_state_dict`` / ``.to(device)`` carry them.  Accepts inputs of any leading shape.

    Residual (multi-codebook) weights: ``indices`` [S, out_features, in_features / v] and ``codebook``
    [S, groups, C, v]; the weight is the running fp16 sum of the S stages' entries (``from_weight(stages=2)``).

    ``index_bits=12``: ``indices`` is the uint8 [out_features, in_features / v * 3/2] tensor ``quantize.pack12``
    makes of 12-bit indices (codebooks of up to 4096 entries at 1.5 bytes per index); ``pack()`` converts a layer
    that holds them in int16.
    """

    def __init__(self, indices: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int = 0,
                 bias: Optional[torch.Tensor] = None, index_bits: Optional[int] = None):
        super().__init__()
        self.packed = index_bits == 12
        if index_bits not in (None, 8, 16, 12):
            raise ValueError("index_bits must be 8, 16 or 12 (packed)")
        if self.packed and (indices.dim() != 2 or indices.dtype != torch.uint8 or indices.shape[1] % 3):
            raise ValueError("packed indices must be a uint8 [N, K/v * 3/2] tensor")
        self.residual = indices.dim() == 3
        if self.residual:
            if codebook.dim() != 4 or codebook.shape[0] != indices.shape[0]:
                raise ValueError("residual weights need indices [S, N, K/v] and codebook [S, G, C, v]")
        elif indices.dim() != 2 or codebook.dim() not in (2, 3):
            raise ValueError("indices must be [N, K/v] and codebook [G, C, v] (or [C, v])")
        if indices.dtype not in (torch.uint8, torch.int16, torch.uint16):
            raise ValueError("indices must be uint8 or (u)int16")
        cb = codebook if codebook.dim() >= 3 else codebook.unsqueeze(0)
        N = indices.shape[-2]
        groups = 1 if rows_per_codebook <= 0 else -(-N // rows_per_codebook)
        if cb.shape[-3] < groups or (self.residual and cb.shape[-3] != groups):
            raise ValueError(f"{cb.shape[-3]} codebooks given, {groups} needed")
        self.out_features = N
        self.v = cb.shape[-1]
        self.in_features = (indices.shape[-1] * 2 // 3 if self.packed else indices.shape[-1]) * self.v
        self.rows_per_codebook = int(rows_per_codebook)
        self.register_buffer("indices", indices.contiguous())
        self.register_buffer("codebook", cb.to(torch.float16).contiguous())
        if bias is not None:
            if bias.shape != (N,):
                raise ValueError("bias must be [out_features]")
            self.register_buffer("bias", bias.to(torch.float16).contiguous())
        else:
            self.bias = None

    @classmethod
    def from_weight(cls, weight: torch.Tensor, *, v: int = 8, entries: int = 256, rows_per_codebook: int = 128,
                    iters: int = 10, seed: int = 0, bias: Optional[torch.Tensor] = None, stages: int = 1) -> "VQLinear":
        """Quantises a dense [out_features, in_features] weight (on its CUDA device) with k-means; ``stages`` > 1
        gives residual weights (every further stage quantises what the stages before it left over)."""
        from .quantize import kmeans_quantize, kmeans_quantize_residual
        if stages > 1:
            idx, cb = kmeans_quantize_residual(weight, stages=stages, v=v, entries=entries, rows_per_codebook=rows_per_codebook,
                                               iters=iters, seed=seed)
        else:
            idx, cb = kmeans_quantize(weight, v=v, entries=entries, rows_per_codebook=rows_per_codebook, iters=iters, seed=seed)
        return cls(idx, cb, rows_per_codebook, bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise RuntimeError(f"last dimension {x.shape[-1]} != in_features {self.in_features}")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype != torch.float16:
            x2 = x2.to(torch.float16)
        op = (torch.ops.vq_gemm_b200.vq_linear_residual if self.residual else
              torch.ops.vq_gemm_b200.vq_linear_packed12 if self.packed else torch.ops.vq_gemm_b200.vq_linear)
        y = op(x2.contiguous(), self.indices, self.codebook, self.rows_per_codebook)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)

    def dequantized_weight(self) -> torch.Tensor:
        """The dense fp16 [out_features, in_features] weight this layer stands for (bit-exact gather)."""
        if self.residual:
            return ops.dequant_residual(self.indices, self.codebook, rows_per_codebook=self.rows_per_codebook)
        return ops.dequant(self.indices, self.codebook, rows_per_codebook=self.rows_per_codebook,
                           index_bits=12 if self.packed else None)

    def pack(self) -> "VQLinear":
        """The same layer with its 12-bit indices (held in int16, at most 4096 entries) packed two to three bytes."""
        from .quantize import pack12
        if self.packed:
            return self
        if self.residual or self.indices.dtype == torch.uint8 or self.codebook.shape[-2] > 4096:
            raise RuntimeError("pack() is for plain weights with int16 indices and at most 4096 entries")
        return VQLinear(pack12(self.indices), self.codebook, self.rows_per_codebook, self.bias, index_bits=12)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, v={self.v}, "
                f"entries={self.codebook.shape[-2]}, rows_per_codebook={self.rows_per_codebook}, "
                f"stages={self.indices.shape[0] if self.residual else 1}, packed12={self.packed}, bias={self.bias is not None}")


class VQGatedUp(nn.Module):
    """First half of a gated MLP with compressed weights: ``SiLU(x W_gate^T) * (x W_up^T)``.

    ``indices`` [2 * intermediate, in_features / v] holds the two projections row-interleaved
    (row 2i = gate row i, row 2i+1 = up row i; ``ops.interleave_gate_up`` builds that order), one
    codebook per ``rows_per_codebook`` of those interleaved rows.  For more than 128 input rows the
    combination happens in the GEMM kernel's epilogue and the two products never reach memory."""

    def __init__(self, indices: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int = 0):
        super().__init__()
        if indices.dim() != 2 or indices.shape[0] % 2 or codebook.dim() not in (2, 3):
            raise ValueError("indices must be [2*N_out, K/v] and codebook [G, C, v] (or [C, v])")
        cb = codebook if codebook.dim() == 3 else codebook.unsqueeze(0)
        self.v = cb.shape[2]
        self.in_features = indices.shape[1] * self.v
        self.out_features = indices.shape[0] // 2
        self.rows_per_codebook = int(rows_per_codebook)
        self.register_buffer("indices", indices.contiguous())
        self.register_buffer("codebook", cb.to(torch.float16).contiguous())

    @classmethod
    def from_weights(cls, gate: torch.Tensor, up: torch.Tensor, *, v: int = 8, entries: int = 256,
                     rows_per_codebook: int = 128, iters: int = 10, seed: int = 0) -> "VQGatedUp":
        """Quantises two dense [intermediate, in_features] fp16 CUDA weights, interleaved, with k-means."""
        from .quantize import kmeans_quantize
        w = ops.interleave_gate_up(gate, up)
        idx, cb = kmeans_quantize(w, v=v, entries=entries, rows_per_codebook=rows_per_codebook, iters=iters, seed=seed)
        return cls(idx, cb, rows_per_codebook)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise RuntimeError(f"last dimension {x.shape[-1]} != in_features {self.in_features}")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype != torch.float16:
            x2 = x2.to(torch.float16)
        y = torch.ops.vq_gemm_b200.vq_swiglu(x2.contiguous(), self.indices, self.codebook, self.rows_per_codebook)
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, v={self.v}, "
                f"entries={self.codebook.shape[1]}, rows_per_codebook={self.rows_per_codebook}")
