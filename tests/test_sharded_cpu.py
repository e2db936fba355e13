"""Host-side logic of the N-sharded mode on CPU: partition arithmetic, weight sharding, and a
world-size-2 gloo run in which each rank computes its column block (with the oracle standing in
for the CUDA kernel) and the all-gathered blocks are interleaved into the full Y."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import vq_oracle as O
from vq_gemm_b200.sharded import interleave_blocks, partition, shard_weights


def test_partition():
    assert partition(28672, 8, 3, 128) == (3 * 3584, 3584)
    assert partition(28672, 1, 0, 128) == (0, 28672)
    assert partition(1024, 2, 1, 0) == (512, 512)
    with pytest.raises(ValueError):
        partition(11008, 4, 0, 128)      # 86 groups do not split 4 ways
    with pytest.raises(ValueError):
        partition(1024, 2, 2, 128)
    assert partition(11008, 2, 1, 128) == (5504, 5504)
    assert partition(768, 2, 0, 192) == (0, 384)   # block must hold whole 192-row groups and 128-column units


def test_shard_weights_cover_the_matrix():
    _, idx, cb = O.make_bl_inputs(1, 64, 1024, 4, 256, 128, seed=0)
    parts = [shard_weights(idx, cb, 4, r, 128) for r in range(4)]
    assert torch.equal(torch.cat([p[0] for p in parts]), idx)
    assert torch.equal(torch.cat([p[1] for p in parts]), cb)
    i0, c0 = shard_weights(idx, cb[:1], 2, 1, 0)    # single codebook: replicated
    assert i0.shape[0] == 512 and c0.shape[0] == 1


def test_interleave_blocks():
    g = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    y = interleave_blocks(g)
    assert y.shape == (3, 8)
    assert torch.equal(y[:, :4], g[0]) and torch.equal(y[:, 4:], g[1])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, M, K, N, v, C, rpc, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=11)
    idx_l, cb_l = shard_weights(idx, cb, world, rank, rpc)
    block = O.vq_gemm_bl(x, idx_l, cb_l, rpc)                 # stand-in for the CUDA kernel
    gathered = torch.empty(world, M, N // world, dtype=torch.float16)
    dist.all_gather_into_tensor(gathered.view(world * M, N // world), block)
    y = interleave_blocks(gathered)
    full = O.vq_gemm_bl(x, idx, cb, rpc)
    q.put((rank, bool(torch.equal(y.view(torch.int16), full.view(torch.int16)))))
    dist.destroy_process_group()


@pytest.mark.parametrize("rpc", [128, 0])
def test_two_rank_gather_equals_single_rank(rpc):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 5, 64, 512, 4, 256, rpc, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)]


def test_k_slices_cover_the_matrix():
    from vq_gemm_b200.sharded import shard_weights_k
    _, idx, _ = O.make_bl_inputs(1, 256, 64, 4, 256, 0, seed=0)
    parts = [shard_weights_k(idx, 4, r) for r in range(4)]
    assert all(p.is_contiguous() and p.shape == (64, 16) for p in parts)
    assert torch.equal(torch.cat(parts, dim=1), idx)
    with pytest.raises(ValueError):
        shard_weights_k(idx, 3, 0)      # 64 index columns do not split 3 ways
    with pytest.raises(ValueError):
        shard_weights_k(idx, 2, 2)


def _rowparallel_worker(rank, world, port, M, K, N, v, C, rpc, q):
    # the row-parallel protocol with the oracle standing in for the CUDA kernels: every rank multiplies its K
    # slice, rounds its partial blocks to fp16, "stores" block o into slot `rank` of owner o (an all-to-all
    # here), and every owner sums its slots in fp32 in rank order
    from vq_gemm_b200.sharded import shard_weights_k
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=13)
    kl = K // world
    partial = O.vq_gemm_bl(x[:, rank * kl:(rank + 1) * kl].contiguous(), shard_weights_k(idx, world, rank), cb, rpc)
    nl = N // world
    send = [partial[:, o * nl:(o + 1) * nl].contiguous() for o in range(world)]
    # gloo has no all_to_all: gather every rank's blocks and pick mine
    everything = [torch.empty(world, M, nl, dtype=torch.float16) for _ in range(world)]
    dist.all_gather(everything, torch.stack(send))
    slots = [everything[r][rank] for r in range(world)]
    acc = torch.zeros(M, nl, dtype=torch.float32)
    for s in slots:
        acc += s.float()
    y_local = acc.half()
    full = O.vq_gemm_bl(x, idx, cb, rpc)[:, rank * nl:(rank + 1) * nl]
    q.put((rank, bool(O.check_tolerance(y_local, full)["ok"])))
    dist.destroy_process_group()


def test_two_rank_row_parallel_reduce_scatter():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rowparallel_worker, args=(r, 2, port, 6, 256, 512, 8, 256, 128, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)]


def _barrier_protocol_worker(rank, world, port, leave_after, q):
    """The epoch-flag protocol of vqg_rank_barrier restated on the host with the process group's store standing in
    for the peer-mapped flag words: arrive = write my epoch into slot `rank` of every other rank's array, wait =
    until every slot of my own array has reached the epoch, bounded in time.  Rank 1 leaves between two steps
    (none of its work in flight); rank 0's next wait runs out, turns into a status code and rank 0 carries on."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    x, idx, cb = O.make_bl_inputs(3, 64, 256, 4, 256, 128, seed=19)
    idx_l, cb_l = shard_weights(idx, cb, world, rank, 128)
    status, log = 0, []
    for epoch in range(1, 5):
        if rank != 0 and epoch > leave_after:
            break                                                   # this rank is gone before step `epoch` starts
        block = O.vq_gemm_bl(x, idx_l, cb_l, 128)                   # the step's work (stand-in for the kernel)
        for r in range(world):
            if r != rank:
                store.set(f"flag/{r}/{rank}/{epoch}", "1")          # arrival at barrier `epoch` in r's array, slot `rank`
        ok = True
        for r in range(world):
            if r != rank:
                try:
                    store.wait([f"flag/{rank}/{r}/{epoch}"], datetime.timedelta(seconds=1.0))
                except Exception:                                   # the bounded wait ran out
                    ok = False
                    status = 11                                     # DS_RANK_BARRIER_TIMEOUT
        log.append((epoch, ok, tuple(block.shape)))
    q.put((rank, status, log))
    # no collective at the end: a rank that left cannot take part in one
    dist.destroy_process_group()


def test_barrier_protocol_when_a_rank_leaves_between_steps():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_barrier_protocol_worker, args=(r, 2, port, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {r: (st, log) for r, st, log in (q.get(timeout=120) for _ in procs)}
    for p in procs:
        p.join(timeout=60)
    st0, log0 = res[0]
    st1, log1 = res[1]
    assert [e for e, ok, _ in log1] == [1, 2] and all(ok for _, ok, _ in log1) and st1 == 0
    assert [ok for _, ok, _ in log0] == [True, True, False, False]   # steps 3 and 4: the other rank never arrives
    assert st0 == 11 and len(log0) == 4                              # rank 0 noticed and still finished every step


def test_lead_slab_is_whole_tiles_and_whole_codebook_groups():
    from types import SimpleNamespace
    from vq_gemm_b200.sharded import ShardedVQGemm
    lead = lambda want, n_local, rpc: ShardedVQGemm._lead(SimpleNamespace(lead_cols=want, n_local=n_local), rpc)
    assert lead(0, 14336, 128) == 0                      # off by default
    assert lead(512, 14336, 128) == 512
    assert lead(600, 14336, 128) == 512                  # rounded down to whole 256-column tiles
    assert lead(512, 1024, 128) == 0                     # more than a quarter of the block: one launch
    assert lead(512, 7168, 0) == 512                     # single codebook
    assert lead(1024, 8192, 384) == 768                  # tiles of 256 and groups of 384 columns meet at 768
    assert lead(256, 4096, 100) == 0                     # no common multiple inside the block
