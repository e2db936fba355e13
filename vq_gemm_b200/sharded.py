"""N-sharded multi-GPU VQ-GEMM: each rank owns a block of output columns (rows of the index
matrix and the codebooks of those rows), X is replicated, and every rank ends up with the whole
Y[M, N].  One process per GPU, ``torch.distributed`` for the plumbing.

Three ways of assembling Y:

``mode="peer"``       Y lives in symmetric memory (two [M, N] buffers per rank, used in turn, peer-mapped
                      over NVLink).  The GEMM epilogue stores each finished tile into every rank's buffer
                      with ordinary global stores (``vqg_gemm_sharded``), so the exchange overlaps the
                      main loop; one bounded barrier across the ranks ends the step (``vqg_rank_barrier``:
                      epoch flags in the same symmetric allocation, a rank that does not arrive within
                      ``barrier_timeout_s`` turns into a status code, not a hang).
``mode="multicast"``  the same, but the epilogue of the prefill kernel issues ONE multimem store per 16
                      bytes to the NVLS multicast mapping of the buffers and the switch replicates it to
                      every rank (``vqg_gemm_sharded_mc``): the SM issues 1/G of the stores and a rank's
                      block leaves its GPU once.  Needs a multicast-capable fabric; ``multicast_available``
                      tells.  Every rank must stay alive while the mapping exists.
``mode="nccl"``       each rank computes its [M, N/G] block, NCCL all-gathers the blocks into
                      [G, M, N/G] and a re-layout copy interleaves them into [M, N].

Lifetime of the returned tensor (peer / multicast): a step writes the buffer that was last written two
steps ago and no barrier precedes the stores, so the tensor returned by a call may be read only by work
that is enqueued ON THE CALLING STREAM BEFORE THE NEXT CALL of the same object.  A reader on another
stream must be waited for (event) before that next call; a reader enqueued after it races with the stores of
ranks that are already one step ahead.  Copy the result if it has to live longer.

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


_FLAG_HALFS = 64          # 128 bytes of epoch flags behind the payload of a symmetric allocation
_SM_HZ = 2.0e9            # cycles per second used to turn a timeout into a cycle limit (upper bound of the SM clock)


class _RankBarrier:
    """Epoch flags of ``vqg_rank_barrier`` inside a symmetric allocation: the last 128 bytes of ``flat``."""

    def __init__(self, flat: torch.Tensor, hdl, world: int, rank: int, timeout_s: float):
        self.world, self.rank = world, rank
        self.flags = flat[-_FLAG_HALFS:].view(torch.int32)
        self.flags.zero_()
        off = (flat.numel() - _FLAG_HALFS) * 2
        self._arr = (ctypes.c_void_p * world)(*[int(p) + off for p in hdl.buffer_ptrs])
        self._limit = int(max(1e3, min(2e10, timeout_s * _SM_HZ)))
        self._epoch = 0
        torch.cuda.current_stream(flat.device).synchronize()
        hdl.barrier()                      # once, at construction: every rank's flags are zero before anyone signals
        torch.cuda.current_stream(flat.device).synchronize()

    def __call__(self, stream: int) -> None:
        self._epoch = (self._epoch + 1) & 0xFFFFFFFF          # flags are compared by signed difference: wrap-around is fine
        st = _lib.load().vqg_rank_barrier(self._arr, self.rank, self.world, self._epoch, self._limit, stream)
        _lib.check(st, "vqg_rank_barrier")


def multicast_available(device: Optional[torch.device] = None, group: Optional[dist.ProcessGroup] = None) -> bool:
    """Whether symmetric memory on this box comes with an NVLS multicast mapping (collective: every rank of
    ``group`` must call it)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) < 2:
        return False
    import torch.distributed._symmetric_memory as symm_mem
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    t = symm_mem.empty(1024, dtype=torch.float16, device=dev)
    hdl = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
    return int(getattr(hdl, "multicast_ptr", 0) or 0) != 0


class ShardedVQGemm:
    """Holds the per-rank output buffers and runs the sharded product.

    Collective construction: every rank of ``group`` must create it with the same M, N and mode."""

    def __init__(self, M: int, N: int, *, group: Optional[dist.ProcessGroup] = None, mode: str = "peer",
                 device: Optional[torch.device] = None, barrier_timeout_s: float = 2.0, lead_cols: int = 0):
        """``lead_cols`` > 0: that many columns of this rank's block are issued as a first launch of their own
        (``vqg_gemm_sharded_cols``), the rest as a second one, so that the first finished tiles cross NVLink
        before the first full wave of tiles is done.  Off by default: measured on 2 GPUs with 512 columns the
        step went from 0.344 to 0.394 ms -- a launch of 16 tiles cut into K pieces over all SMs pays more for
        summing the pieces than the earlier start of the stream returns."""
        if mode not in ("peer", "multicast", "nccl"):
            raise ValueError("mode must be 'peer', 'multicast' or 'nccl'")
        self.lead_cols = lead_cols
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
        self._mc = 0
        if self.world == 1:
            self.y = torch.empty((M, N), dtype=torch.float16, device=self.device)
            self._ptrs = [self.y.data_ptr()]
        elif mode in ("peer", "multicast"):
            import torch.distributed._symmetric_memory as symm_mem
            self._flat = symm_mem.empty(2 * M * N + _FLAG_HALFS, dtype=torch.float16, device=self.device)
            self._hdl = symm_mem.rendezvous(self._flat, self.group)
            self._ybuf = self._flat[:2 * M * N].view(2, M, N)
            self._ptrs = [int(p) for p in self._hdl.buffer_ptrs]
            if self._ptrs[self.rank] != self._flat.data_ptr():
                raise RuntimeError("symmetric memory: local buffer pointer mismatch")
            if mode == "multicast":
                self._mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
                if self._mc == 0:
                    raise RuntimeError("symmetric memory has no multicast mapping on this machine (mode='peer' works without)")
            self._barrier = _RankBarrier(self._flat, self._hdl, self.world, self.rank, barrier_timeout_s)
            self._step = 0
            self.y = self._ybuf[0]
        else:
            self.y = torch.empty((M, N), dtype=torch.float16, device=self.device)
            self._block = torch.empty((M, self.n_local), dtype=torch.float16, device=self.device)
            self._gathered = torch.empty((self.world, M, self.n_local), dtype=torch.float16, device=self.device)
        self._ws = None
        self._retired = []
        self._plans = {}

    def _lead(self, rows_per_codebook: int) -> int:
        """Columns of the small first launch: whole 256-column tiles and whole codebook groups, at most a quarter
        of the block."""
        want = self.lead_cols or 0
        unit = 256
        if rows_per_codebook > 0:
            while unit % rows_per_codebook:
                unit += 256
                if unit > self.n_local:
                    return 0
        want = want // unit * unit
        return want if 0 < want <= self.n_local // 4 else 0

    def _ws_bytes(self, lib, M, K, v, C, ib, rows_per_codebook) -> int:
        lead = self._lead(rows_per_codebook) if self.world > 1 else 0
        return max(lib.vqg_workspace_bytes(M, n, K, v, C, ib, rows_per_codebook, _lib.LAYOUT_BL, _lib.PATH_AUTO)
                   for n in ((lead, self.n_local - lead) if lead else (self.n_local,)))

    def _workspace(self, nbytes: int):
        if nbytes == 0:
            return None, 0
        if self._ws is None or self._ws.numel() < nbytes:
            if self._ws is not None:
                self._retired.append(self._ws)   # a captured graph may still hold its address
            self._ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        return self._ws.data_ptr(), self._ws.numel()

    def gather_x(self, x_rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """All-gather of a row-sharded activation: every rank passes its [M/G, K] block of X (rank r holds rows
        [r*M/G, (r+1)*M/G)) and gets the whole [M, K] back.  Lets a host feed each GPU 1/G of X instead of all of it."""
        if self.world == 1:
            return x_rows
        if out is None:
            out = torch.empty((x_rows.shape[0] * self.world, x_rows.shape[1]), dtype=x_rows.dtype, device=x_rows.device)
        dist.all_gather_into_tensor(out, x_rows.contiguous(), group=self.group)
        return out

    def __call__(self, x: torch.Tensor, idx_local: torch.Tensor, cb_local: torch.Tensor, rows_per_codebook: int = 0,
                 copy: bool = False):
        """x [M, K] (replicated), idx_local [N/G, K/v], cb_local: the block's codebooks.  Returns the rank's full
        Y[M, N]: valid for work enqueued on the current stream before the next call of this object (see the
        module text); with ``copy=True`` a private copy that stays valid."""
        y = self._run(x, idx_local, cb_local, rows_per_codebook)
        return y.clone() if copy else y

    def _run(self, x: torch.Tensor, idx_local: torch.Tensor, cb_local: torch.Tensor, rows_per_codebook: int = 0):
        lib = _lib.load()
        M, K = x.shape
        if M != self.M or idx_local.shape[0] != self.n_local:
            raise RuntimeError("shapes do not match the buffers this object was built for")
        cb3 = cb_local if cb_local.dim() == 3 else cb_local.unsqueeze(0)
        _, C, v = cb3.shape
        ib = 1 if idx_local.dtype == torch.uint8 else 2
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if self.mode != "nccl" or self.world == 1:
            # per-shape constants are looked up once: at 8 ranks a step is ~0.2 ms and host time counts
            key = (K, v, C, ib, rows_per_codebook)
            plan = self._plans.get(key)
            if plan is None:
                nbytes = self._ws_bytes(lib, M, K, v, C, ib, rows_per_codebook)
                arrs = [(ctypes.c_void_p * self.world)(*[p + par * self.M * self.N * 2 for p in self._ptrs])
                        for par in range(2 if self._hdl is not None else 1)]
                plan = self._plans[key] = (nbytes, arrs)
            nbytes, arrs = plan
            ws_ptr, ws_n = self._workspace(nbytes)   # looked up every call: the buffer may have been regrown
            arr, mc = arrs[0], None
            if self._hdl is not None:
                par = self._step & 1
                self.y = self._ybuf[par]
                arr = arrs[par]
                if self._mc:
                    mc = self._mc + par * self.M * self.N * 2
                self._step += 1
            lead = self._lead(rows_per_codebook) if self.world > 1 else 0
            col0 = self.rank * self.n_local
            if lead:
                # slab 1: the first `lead` columns (their indices are the first rows of the shard, their codebooks
                # the first groups); slab 2: the rest.  Same workspace, stream order.
                g = lead // rows_per_codebook if rows_per_codebook > 0 else 0
                st = lib.vqg_gemm_sharded_cols(x.data_ptr(), idx_local.data_ptr(), cb_local.data_ptr(), arr, mc, self.rank,
                                               self.world, M, lead, K, v, C, ib, rows_per_codebook, col0, self.N,
                                               ws_ptr, ws_n, stream)
                _lib.check(st, "vqg_gemm_sharded_cols")
                st = lib.vqg_gemm_sharded_cols(x.data_ptr(), idx_local[lead:].data_ptr(), cb3[g:].data_ptr(), arr, mc,
                                               self.rank, self.world, M, self.n_local - lead, K, v, C, ib, rows_per_codebook,
                                               col0 + lead, self.N, ws_ptr, ws_n, stream)
            else:
                st = lib.vqg_gemm_sharded_cols(x.data_ptr(), idx_local.data_ptr(), cb_local.data_ptr(), arr, mc, self.rank,
                                               self.world, M, self.n_local, K, v, C, ib, rows_per_codebook, col0, self.N,
                                               ws_ptr, ws_n, stream)
            _lib.check(st, "vqg_gemm_sharded_cols")
            if self._hdl is not None:
                self._barrier(stream)   # every rank's stores into this rank's buffer have landed
            return self.y
        # the block is computed in the same launches as in the fused modes (same K cuts, hence the same bits)
        lead = self._lead(rows_per_codebook)
        ws_ptr, ws_n = self._workspace(self._ws_bytes(lib, M, K, v, C, ib, rows_per_codebook))
        own = (ctypes.c_void_p * 1)(self._block.data_ptr())
        g = lead // rows_per_codebook if (lead and rows_per_codebook > 0) else 0
        for c0, cols, ip, cp in ((0, lead, idx_local, cb_local), (lead, self.n_local - lead, idx_local[lead:], cb3[g:])):
            if cols:
                st = lib.vqg_gemm_sharded_cols(x.data_ptr(), ip.data_ptr(), cp.data_ptr(), own, None, 0, 1, M, cols, K, v, C, ib,
                                               rows_per_codebook, c0, self.n_local, ws_ptr, ws_n, stream)
                _lib.check(st, "vqg_gemm_sharded_cols")
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

    def __init__(self, M: int, N: int, *, group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 barrier_timeout_s: float = 2.0):
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
            self._flat = symm_mem.empty(2 * G * M * self.n_local + _FLAG_HALFS, dtype=torch.float16, device=self.device)
            self._hdl = symm_mem.rendezvous(self._flat, self.group)
            self._part = self._flat[:2 * G * M * self.n_local].view(2, G, M, self.n_local)
            self._bases = [int(p) for p in self._hdl.buffer_ptrs]
            if self._bases[self.rank] != self._flat.data_ptr():
                raise RuntimeError("symmetric memory: local buffer pointer mismatch")
            self._barrier = _RankBarrier(self._flat, self._hdl, G, self.rank, barrier_timeout_s)
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
            self._barrier(stream)   # every rank's partial of my block has landed in my slots
        st = lib.vqg_reduce_slots(self._part[par].data_ptr(), self.y.data_ptr(), self.world, M, self.n_local, self.n_local, stream)
        _lib.check(st, "vqg_reduce_slots")
        return self.y
