"""N-sharded multi-GPU VQ-GEMM: each rank owns a block of output columns (rows of the index
matrix and the codebooks of those rows), X is replicated, and every rank ends up with the whole
Y[M, N].  One process per GPU, ``torch.distributed`` for the plumbing.

Two ways of assembling Y:

``mode="peer"``   Y lives in symmetric memory (two [M, N] buffers per rank, used in turn, peer-mapped
                  over NVLink).  The GEMM epilogue stores each finished tile into every rank's buffer
                  with ordinary global stores (``vqg_gemm_sharded``), so the exchange overlaps the
                  main loop; one device-side barrier across ranks ends the step.  A step writes the
                  buffer that was last written two steps ago: every rank passed the previous step's
                  barrier after reading it, so no barrier is needed before the stores.  The returned
                  tensor is therefore valid until the second call after it.  No TMA and no multicast
                  touch peer memory.
``mode="nccl"``   each rank computes its [M, N/G] block, NCCL all-gathers the blocks into
                  [G, M, N/G] and a re-layout copy interleaves them into [M, N].

``RowParallelVQGemm`` is the K-sharded counterpart for the second half of a tensor-parallel MLP:
each rank multiplies its slice of the input features by its K slice of the weights, the partial
[M, N/G] blocks go straight to their owners (TMA tensor stores from the GEMM epilogue into slot
``rank`` of the owner's symmetric buffer), one barrier, and every owner sums its G slots: a fused
GEMM + reduce-scatter.  With the N-sharded first half leaving its output on the rank that
computed it, the intermediate activation is never gathered.

The reference has no multi-GPU code (device 0 is hard-coded, strategy_1/src.cu:343).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib


def partition(N: int, world: int, rank: int, rows_per_codebook: int = 0, align: int = 128) -> Tuple[int, int]:
    """Column block ``(row0, n_local)`` of rank ``rank``: equal blocks, each a whole number of
    codebook groups and of ``align`` columns.  Raises if N does not split that way."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank / world size")
    unit = math.lcm(align, rows_per_codebook) if rows_per_codebook > 0 else align
    if N % (world * unit):
        raise ValueError(f"N={N} does not split into {world} blocks of a multiple of {unit} columns")
    n_local = N // world
    return rank * n_local, n_local


def shard_weights(idx: torch.Tensor, codebook: torch.Tensor, world: int, rank: int, rows_per_codebook: int):
    """Slices a full (idx [N, K/v], codebook [G, C, v]) pair down to the rank's block."""
    N = idx.shape[0]
    row0, n_local = partition(N, world, rank, rows_per_codebook)
    if rows_per_codebook <= 0:
        return idx[row0:row0 + n_local].contiguous(), codebook  # one codebook: every rank holds it
    g0 = row0 // rows_per_codebook
    return (idx[row0:row0 + n_local].contiguous(),
            codebook[g0:g0 + n_local // rows_per_codebook].contiguous())


def interleave_blocks(gathered: torch.Tensor) -> torch.Tensor:
    """[G, M, n_local] (what an all-gather of column blocks yields) -> [M, G*n_local]."""
    G, M, n_local = gathered.shape
    return gathered.permute(1, 0, 2).reshape(M, G * n_local)


class ShardedVQGemm:
    """Holds the per-rank output buffers and runs the sharded product.

    Collective construction: every rank of ``group`` must create it with the same M and N."""

    def __init__(self, M: int, N: int, *, group: Optional[dist.ProcessGroup] = None, mode: str = "peer",
                 device: Optional[torch.device] = None):
        if mode not in ("peer", "nccl"):
            raise ValueError("mode must be 'peer' or 'nccl'")
        if dist.is_available() and dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self.world = dist.get_world_size(self.group)
            self.rank = dist.get_rank(self.group)
        else:  # single process: behaves as a world of one
            self.group, self.world, self.rank = None, 1, 0
        self.M, self.N, self.mode = M, N, mode
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        if N % self.world:
            raise ValueError("N must be a multiple of the world size")
        self.n_local = N // self.world
        self._hdl = None
        if self.world == 1:
            self.y = torch.empty((M, N), dtype=torch.float16, device=self.device)
            self._ptrs = [self.y.data_ptr()]
        elif mode == "peer":
            import torch.distributed._symmetric_memory as symm_mem
            self._ybuf = symm_mem.empty((2, M, N), dtype=torch.float16, device=self.device)
            self._hdl = symm_mem.rendezvous(self._ybuf, self.group)
            self._ptrs = [int(p) for p in self._hdl.buffer_ptrs]
            if self._ptrs[self.rank] != self._ybuf.data_ptr():
                raise RuntimeError("symmetric memory: local buffer pointer mismatch")
            self._step = 0
            self.y = self._ybuf[0]
        else:
            self.y = torch.empty((M, N), dtype=torch.float16, device=self.device)
            self._block = torch.empty((M, self.n_local), dtype=torch.float16, device=self.device)
            self._gathered = torch.empty((self.world, M, self.n_local), dtype=torch.float16, device=self.device)
        self._ws = None
        self._retired = []
        self._plans = {}

    def _workspace(self, nbytes: int):
        if nbytes == 0:
            return None, 0
        if self._ws is None or self._ws.numel() < nbytes:
            if self._ws is not None:
                self._retired.append(self._ws)   # a captured graph may still hold its address
            self._ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        return self._ws.data_ptr(), self._ws.numel()

    def __call__(self, x: torch.Tensor, idx_local: torch.Tensor, cb_local: torch.Tensor, rows_per_codebook: int = 0):
        """x [M, K] (replicated), idx_local [N/G, K/v], cb_local: the block's codebooks.  Returns
        the rank's full Y[M, N]; valid after the call on the current stream."""
        lib = _lib.load()
        M, K = x.shape
        if M != self.M or idx_local.shape[0] != self.n_local:
            raise RuntimeError("shapes do not match the buffers this object was built for")
        cb3 = cb_local if cb_local.dim() == 3 else cb_local.unsqueeze(0)
        _, C, v = cb3.shape
        ib = 1 if idx_local.dtype == torch.uint8 else 2
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if self.mode == "peer" or self.world == 1:
            # per-shape constants are looked up once: at 8 ranks a step is ~0.2 ms and host time counts
            key = (K, v, C, ib, rows_per_codebook)
            plan = self._plans.get(key)
            if plan is None:
                nbytes = lib.vqg_workspace_bytes(M, self.n_local, K, v, C, ib, rows_per_codebook, _lib.LAYOUT_BL, _lib.PATH_AUTO)
                arrs = [(ctypes.c_void_p * self.world)(*[p + par * self.M * self.N * 2 for p in self._ptrs])
                        for par in range(2 if self._hdl is not None else 1)]
                plan = self._plans[key] = (nbytes, arrs)
            nbytes, arrs = plan
            ws_ptr, ws_n = self._workspace(nbytes)   # looked up every call: the buffer may have been regrown
            arr = arrs[0]
            if self._hdl is not None:
                par = self._step & 1
                self.y = self._ybuf[par]
                arr = arrs[par]
                self._step += 1
            st = lib.vqg_gemm_sharded(x.data_ptr(), idx_local.data_ptr(), cb_local.data_ptr(), arr, self.rank,
                                      self.world, M, self.n_local, K, v, C, ib, rows_per_codebook, ws_ptr, ws_n, stream)
            _lib.check(st, "vqg_gemm_sharded")
            if self._hdl is not None:
                self._hdl.barrier()  # every rank's stores into this rank's buffer have landed
            return self.y
        from .ops import vq_gemm
        vq_gemm(x, idx_local, cb_local, rows_per_codebook=rows_per_codebook, layout="bl", out=self._block)
        dist.all_gather_into_tensor(self._gathered.view(self.world * M, self.n_local), self._block, group=self.group)
        self.y.copy_(interleave_blocks(self._gathered))
        return self.y


def shard_weights_k(idx: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """K slice of an index matrix [N, K/v] for the row-parallel product: columns
    ``[rank * J/G, (rank + 1) * J/G)`` with ``J = K/v``, as a contiguous copy."""
    J = idx.shape[1]
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank / world size")
    if J % world:
        raise ValueError(f"K/v = {J} does not split into {world} equal slices")
    j = J // world
    return idx[:, rank * j:(rank + 1) * j].contiguous()


class RowParallelVQGemm:
    """Fused K-sharded product + reduce-scatter: ``y_local[M, N/G] = (sum_r x_r @ W_r^T)[:, block of this rank]``.

    Collective construction (same M and N on every rank of ``group``).  The per-rank partial blocks
    live in symmetric memory as two sets of G slots used in turn, so that one barrier per step (after
    the stores, before the sum) is enough."""

    def __init__(self, M: int, N: int, *, group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None):
        if dist.is_available() and dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self.world = dist.get_world_size(self.group)
            self.rank = dist.get_rank(self.group)
        else:
            self.group, self.world, self.rank = None, 1, 0
        if N % (self.world * 128):
            raise ValueError(f"N={N} does not split into {self.world} blocks of a multiple of 128 columns")
        self.M, self.N, self.n_local = M, N, N // self.world
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._hdl = None
        G = self.world
        if G == 1:
            self._part = torch.empty((1, 1, M, N), dtype=torch.float16, device=self.device)
            self._bases = [self._part.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self._part = symm_mem.empty((2, G, M, self.n_local), dtype=torch.float16, device=self.device)
            self._hdl = symm_mem.rendezvous(self._part, self.group)
            self._bases = [int(p) for p in self._hdl.buffer_ptrs]
            if self._bases[self.rank] != self._part.data_ptr():
                raise RuntimeError("symmetric memory: local buffer pointer mismatch")
        self.y = torch.empty((M, self.n_local), dtype=torch.float16, device=self.device)
        self._step = 0
        self._ws = None
        self._retired = []
        slot_bytes = M * self.n_local * 2
        self._arrs = [(ctypes.c_void_p * G)(*[b + (par * G + self.rank) * slot_bytes for b in self._bases])
                      for par in range(2 if G > 1 else 1)]

    def __call__(self, x_local: torch.Tensor, idx_local: torch.Tensor, codebook: torch.Tensor, rows_per_codebook: int = 0):
        """x_local [M, K/G], idx_local [N, K/(G v)] (``shard_weights_k``), codebook: all groups.  Returns this
        rank's block of the summed product; valid after the call on the current stream."""
        lib = _lib.load()
        M, K_local = x_local.shape
        if M != self.M or idx_local.shape[0] != self.N:
            raise RuntimeError("shapes do not match the buffers this object was built for")
        cb3 = codebook if codebook.dim() == 3 else codebook.unsqueeze(0)
        _, C, v = cb3.shape
        ib = 1 if idx_local.dtype == torch.uint8 else 2
        stream = torch.cuda.current_stream(self.device).cuda_stream
        nbytes = lib.vqg_rowparallel_workspace_bytes(M, self.N, K_local, v, C, ib, rows_per_codebook)
        if nbytes and (self._ws is None or self._ws.numel() < nbytes):
            if self._ws is not None:
                self._retired.append(self._ws)   # a captured graph may still hold its address
            self._ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        par = (self._step & 1) if self.world > 1 else 0
        self._step += 1
        st = lib.vqg_gemm_rowparallel(x_local.data_ptr(), idx_local.data_ptr(), codebook.data_ptr(), self._arrs[par], self.world,
                                      M, self.N, K_local, v, C, ib, rows_per_codebook,
                                      self._ws.data_ptr() if nbytes else None, self._ws.numel() if nbytes else 0, stream)
        _lib.check(st, "vqg_gemm_rowparallel")
        if self._hdl is not None:
            self._hdl.barrier()   # every rank's partial of my block has landed in my slots
        st = lib.vqg_reduce_slots(self._part[par].data_ptr(), self.y.data_ptr(), self.world, M, self.n_local, self.n_local, stream)
        _lib.check(st, "vqg_reduce_slots")
        return self.y
