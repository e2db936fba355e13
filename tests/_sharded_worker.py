"""Worker for tests/test_gpu_sharded.py (one process per GPU, started by torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import vq_gemm_b200 as V  # noqa: E402
from oracle import vq_oracle as O  # noqa: E402
from vq_gemm_b200.sharded import ShardedVQGemm, shard_weights  # noqa: E402


def rowparallel(rank, world, dev):
    """K-sharded product + reduce-scatter against the oracle's column block; three steps in a row reuse the
    alternating slot sets and must give the same bits."""
    from vq_gemm_b200.sharded import RowParallelVQGemm, shard_weights_k
    ok = True
    for (M, K, N, v, C, rpc) in [(300, 2048, 512, 8, 256, 128), (24, 1024, 256, 4, 256, 128), (1024, 4096, 1024, 8, 256, 128)]:
        x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=17)
        kl, nl = K // world, N // world
        op = RowParallelVQGemm(M, N, device=dev)
        xl = x[:, rank * kl:(rank + 1) * kl].contiguous().to(dev)
        il = shard_weights_k(idx, world, rank).to(dev)
        outs = [op(xl, il, cb.to(dev), rpc).clone() for _ in range(3)]
        torch.cuda.synchronize()
        ref = O.vq_gemm_bl(x, idx, cb, rpc)[:, rank * nl:(rank + 1) * nl]
        tol = O.check_tolerance(outs[0].cpu(), ref)["ok"]
        same = all(torch.equal(o.view(torch.int16), outs[0].view(torch.int16)) for o in outs[1:])
        if not (tol and same):
            ok = False
            print(f"rank {rank}: ROWPARALLEL MISMATCH shape={(M, K, N, v)} tol={tol} deterministic={same}", flush=True)
    return ok


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    cases = [(256, 512, 1024, 4, 256, 128), (4, 1024, 512, 8, 256, 128), (512, 1024, 2048, 8, 256, 128)]
    if os.environ.get("VQG_WORKER_MODE") == "rowparallel":
        ok = rowparallel(rank, world, dev)
        cases = []
    modes = ["peer", "nccl"]
    if cases and os.environ.get("VQG_WORKER_MULTICAST") == "1":
        from vq_gemm_b200.sharded import multicast_available
        if multicast_available(dev):
            modes.append("multicast")
            if rank == 0:
                print("MULTICAST_TESTED", flush=True)
    if cases:
        # a row-sharded activation all-gathered over NVLink equals the whole
        xs = torch.arange(64 * 96, dtype=torch.float16).reshape(64, 96)
        m_rows = 64 // world
        got = ShardedVQGemm(64, 256 * world, mode="nccl", device=dev).gather_x(xs[rank * m_rows:(rank + 1) * m_rows].to(dev))
        if not torch.equal(got.cpu(), xs):
            ok = False
            print(f"rank {rank}: gather_x MISMATCH", flush=True)
    for (M, K, N, v, C, rpc) in cases:
        x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=5)
        # the single-GPU result, block by block: a block computed alone has the same shape, hence the same
        # schedule and summation order, as the one a rank computes (the whole-N product may cut its K loops
        # elsewhere and differ in the last bits)
        blocks = []
        for r in range(world):
            idx_r, cb_r = shard_weights(idx, cb, world, r, rpc)
            blocks.append(V.vq_gemm(x.to(dev), idx_r.to(dev), cb_r.to(dev), rows_per_codebook=rpc, layout="bl"))
        single = torch.cat(blocks, dim=1)
        idx_l, cb_l = shard_weights(idx, cb, world, rank, rpc)
        for mode in modes:
            op = ShardedVQGemm(M, N, mode=mode, device=dev)
            for _ in range(3):
                y = op(x.to(dev), idx_l.to(dev), cb_l.to(dev), rpc)
            torch.cuda.synchronize()
            same = bool(torch.equal(y.view(torch.int16), single.view(torch.int16)))
            tol = O.check_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, rpc))["ok"]
            if not (same and tol):
                ok = False
                print(f"rank {rank}: MISMATCH mode={mode} shape={(M, K, N, v)} bitwise={same} tol={tol}", flush=True)
    if cases:
        # a block issued as two launches (a 256-column first slab): every fused mode equals the NCCL mode bit for bit
        # (which computes in the same two launches) and the oracle within the tolerance
        M, K, N, v, C, rpc = 256, 512, 1024 * world, 8, 256, 128
        x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=9)
        idx_l, cb_l = shard_weights(idx, cb, world, rank, rpc)
        ref = None
        for mode in ["nccl"] + [m for m in modes if m != "nccl"]:
            op = ShardedVQGemm(M, N, mode=mode, device=dev, lead_cols=256)
            assert op._lead(rpc) == 256
            for _ in range(2):
                y = op(x.to(dev), idx_l.to(dev), cb_l.to(dev), rpc)
            torch.cuda.synchronize()
            if ref is None:
                ref = y.clone()
                if not O.check_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, rpc))["ok"]:
                    ok = False
                    print(f"rank {rank}: slab launches out of tolerance", flush=True)
            elif not torch.equal(y.view(torch.int16), ref.view(torch.int16)):
                ok = False
                print(f"rank {rank}: slab launches MISMATCH mode={mode}", flush=True)
    ok = ok and V.device_status() == 0
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("SHARDED_OK" if int(t.item()) == 1 else "SHARDED_FAIL", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(t.item()) == 1 else 1)


if __name__ == "__main__":
    main()
