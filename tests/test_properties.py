"""Property-based checks (hypothesis) of the CPU restatements and the host-side layout helpers:
random small shapes instead of a fixed list.  No GPU."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from oracle import quantize_oracle as Q
from oracle import vq_oracle as O
from vq_gemm_b200.ops import interleave_gate_up
from vq_gemm_b200.sharded import interleave_blocks, partition, shard_weights, shard_weights_k

SET = dict(max_examples=25, deadline=None)


@settings(**SET)
@given(v=st.sampled_from([1, 2, 4, 8]), j=st.integers(1, 6), n=st.integers(1, 12), c=st.integers(1, 300),
       rpc=st.sampled_from([0, 1, 3, 4]), seed=st.integers(0, 2 ** 16))
def test_vectorised_gather_equals_the_scalar_rule(v, j, n, c, rpc, seed):
    g = torch.Generator().manual_seed(seed)
    groups = 1 if rpc <= 0 else -(-n // rpc)
    cb = torch.randn(groups, c, v, generator=g).half()
    dt = torch.uint8 if c <= 256 else torch.int16
    idx = torch.randint(0, c, (n, j), generator=g).to(dt)
    assert torch.equal(O.dequant_bl_layout(idx, cb, rpc).view(torch.int16), O.dequant_bl_scalar(idx, cb, rpc).view(torch.int16))


@settings(**SET)
@given(m=st.integers(1, 5), v=st.sampled_from([2, 4, 8]), j=st.integers(1, 5), n=st.integers(1, 10), seed=st.integers(0, 2 ** 16))
def test_product_is_linear_in_x_and_splits_over_k(m, v, j, n, seed):
    g = torch.Generator().manual_seed(seed)
    k = v * j
    x = torch.randn(m, k, generator=g).half()
    cb = (torch.randn(1, 64, v, generator=g) * 0.1).half()
    idx = torch.randint(0, 64, (n, j), generator=g).to(torch.uint8)
    w = O.dequant_bl_layout(idx, cb, 0).float()
    full = x.float() @ w.t()
    # the K split of the row-parallel mode: partial products over index-column slices add up
    cut = (j // 2) * v
    parts = x[:, :cut].float() @ w[:, :cut].t() + x[:, cut:].float() @ w[:, cut:].t()
    assert torch.allclose(parts, full, atol=1e-4, rtol=1e-4)
    assert O.check_tolerance(O.vq_gemm_bl(x, idx, cb, 0), full.half())["ok"]


@settings(**SET)
@given(world=st.sampled_from([1, 2, 4, 8]), blocks=st.integers(1, 3), rpc=st.sampled_from([0, 128, 256]), j=st.integers(1, 4))
def test_column_and_k_partitions_tile_the_matrix(world, blocks, rpc, j):
    unit = max(rpc, 128) if rpc else 128
    n = world * blocks * unit
    idx = torch.arange(n * j * world, dtype=torch.int32).reshape(n, j * world)
    groups = 1 if rpc == 0 else n // rpc
    cb = torch.zeros(groups, 4, 2, dtype=torch.float16)
    rows = [shard_weights(idx, cb, world, r, rpc)[0] for r in range(world)]
    assert torch.equal(torch.cat(rows), idx)
    assert [partition(n, world, r, rpc)[0] for r in range(world)] == [r * n // world for r in range(world)]
    cols = [shard_weights_k(idx, world, r) for r in range(world)]
    assert torch.equal(torch.cat(cols, dim=1), idx)
    gathered = torch.stack([torch.full((3, n // world), float(r)) for r in range(world)])
    y = interleave_blocks(gathered)
    assert y.shape == (3, n) and all(bool((y[:, r * n // world:(r + 1) * n // world] == r).all()) for r in range(world))


@settings(**SET)
@given(n=st.integers(1, 9), k=st.integers(1, 5), seed=st.integers(0, 2 ** 16))
def test_gate_up_interleave_round_trip(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a, b = torch.randn(n, k, generator=g), torch.randn(n, k, generator=g)
    w = interleave_gate_up(a, b)
    assert torch.equal(w[0::2], a) and torch.equal(w[1::2], b)


@settings(**SET)
@given(rows=st.integers(1, 6), pairs=st.integers(1, 40), seed=st.integers(0, 2 ** 16))
def test_pack12_round_trip(rows, pairs, seed):
    rng = np.random.default_rng(seed)
    idx = rng.integers(0, 4096, size=(rows, 2 * pairs)).astype(np.int16)
    p = Q.pack12(idx)
    assert p.shape == (rows, 3 * pairs)
    assert np.array_equal(Q.unpack12(p), idx)


@settings(**SET)
@given(v=st.sampled_from([2, 4, 8]), c=st.integers(1, 40), n=st.integers(1, 8), j=st.integers(1, 4), seed=st.integers(0, 2 ** 16))
def test_assign_is_idempotent_and_never_worse_than_any_entry(v, c, n, j, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, v * j)) * 0.1).astype(np.float16)
    cb = (rng.standard_normal((1, c, v)) * 0.1).astype(np.float16)
    idx = Q.assign(w, cb, 0)
    deq = cb[0][idx.astype(np.int64).reshape(-1)].reshape(n, v * j)
    assert np.array_equal(cb[0][Q.assign(deq, cb, 0).astype(np.int64).reshape(-1)].reshape(n, v * j), deq)
    sub = w.astype(np.float32).reshape(-1, v)
    chosen = ((sub - cb[0].astype(np.float32)[idx.reshape(-1).astype(np.int64)]) ** 2).sum(1)
    every = ((sub[:, None, :] - cb[0].astype(np.float32)[None]) ** 2).sum(2)
    assert np.all(chosen <= every.min(1) + 1e-6)
    # one Lloyd step does not raise the distortion beyond fp16 rounding of the centroids
    new = Q.update(w, idx, cb, 0)
    assert Q.distortion(w, idx, new, 0) <= Q.distortion(w, idx, cb, 0) * (1 + 1e-2) + 1e-9
