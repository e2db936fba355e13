"""Weight formats, layout inference, synthetic inputs and algorithmic byte / flop counts.

Two formats (see include/vqg.h): ``"bl"`` -- indices ``[N, K/v]``, codebook ``[G, C, v]`` with one
codebook per ``rows_per_codebook`` output rows; ``"ref"`` -- the reference's own format, indices
``[K, Nq]`` uint8, codebook ``[Nq/4, 256, 2]`` (reference bench.py:29-30,83-85).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class VQShape:
    """One benchmark configuration."""
    name: str
    M: int
    K: int
    N: int
    v: int
    C: int
    rows_per_codebook: int  # 0 = one codebook for the matrix
    idx_bytes: int
    bound: str              # "hbm" or "tensor"

    @property
    def groups(self) -> int:
        return 1 if self.rows_per_codebook <= 0 else (self.N + self.rows_per_codebook - 1) // self.rows_per_codebook

    @property
    def flops(self) -> int:
        return 2 * self.M * self.N * self.K

    @property
    def bytes_idx(self) -> int:
        return self.N * (self.K // self.v) * self.idx_bytes

    @property
    def bytes_codebook(self) -> int:
        return self.groups * self.C * self.v * 2

    @property
    def bytes_algorithmic(self) -> int:
        """Compressed traffic: indices + codebooks + X + Y (never the dequantised weights)."""
        return self.bytes_idx + self.bytes_codebook + 2 * self.M * self.K + 2 * self.M * self.N


# The five configurations of the benchmark contract, in order.
CONFIGS = {
    "c1_cpu_ref": VQShape("c1_cpu_ref", 16, 4096, 4096, 4, 256, 0, 1, "hbm"),
    "c2_decode": VQShape("c2_decode", 1, 4096, 11008, 4, 256, 128, 1, "hbm"),
    "c3_small_batch": VQShape("c3_small_batch", 16, 8192, 8192, 8, 4096, 0, 2, "hbm"),
    "c4_prefill": VQShape("c4_prefill", 4096, 4096, 14336, 4, 256, 128, 1, "tensor"),
    "c5_mlp70b": VQShape("c5_mlp70b", 2048, 8192, 28672, 8, 256, 128, 1, "tensor"),
}


def make_inputs(shape: VQShape, seed: int = 0, device="cpu", n_rows: Optional[int] = None, row0: int = 0):
    """Seeded synthetic inputs for a configuration: X fp16 ~ N(0,1), codebook fp16 ~ N(0,0.02),
    indices uniform in [0, C).  ``n_rows``/``row0`` select a block of output rows (a shard)
    without materialising the rest; blocks must be aligned to codebook groups."""
    N = shape.N if n_rows is None else n_rows
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape.M, shape.K, generator=g).half()
    rpc = shape.rows_per_codebook
    if rpc > 0:
        assert row0 % rpc == 0 and N % rpc == 0
        G = N // rpc
    else:
        assert n_rows is None
        G = 1
    gs = torch.Generator().manual_seed(seed * 7919 + 13 + row0)
    cb = (torch.randn(G, shape.C, shape.v, generator=gs) * 0.02).half()
    idx = torch.randint(0, shape.C, (N, shape.K // shape.v), generator=gs, dtype=torch.int32)
    idx = idx.to(torch.uint8) if shape.idx_bytes == 1 else idx.to(torch.int16)
    return x.to(device), idx.to(device), cb.to(device)


def infer_layout(x: torch.Tensor, indices: torch.Tensor, codebook: torch.Tensor) -> str:
    """Decides between the two formats from the shapes alone; ambiguous or inconsistent shapes raise."""
    if x.dim() != 2 or indices.dim() != 2 or codebook.dim() not in (2, 3):
        raise RuntimeError("vq_gemm expects x [M,K], indices 2-D, codebook [G,C,v] or [C,v]")
    K = x.shape[1]
    v = codebook.shape[-1]
    is_bl = indices.shape[1] * v == K
    is_ref = (codebook.dim() == 3 and v == 2 and indices.shape[0] == K and indices.shape[1] % 4 == 0
              and codebook.shape[0] == indices.shape[1] // 4 and codebook.shape[1] == 256
              and indices.dtype == torch.uint8)
    if is_ref and not is_bl:
        return "ref"
    if is_bl and not is_ref:
        return "bl"
    if is_bl and is_ref:
        raise RuntimeError("shapes fit both weight formats; pass layout='bl' or layout='ref'")
    raise RuntimeError(
        f"shapes fit neither weight format: x {tuple(x.shape)}, indices {tuple(indices.shape)}, "
        f"codebook {tuple(codebook.shape)}")
