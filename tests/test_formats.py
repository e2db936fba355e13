"""Host logic: layout inference, configuration table, shard-aligned input generation."""
import pytest
import torch

import vq_gemm_b200 as V
from vq_gemm_b200.formats import CONFIGS, infer_layout, make_inputs


def test_config_table_matches_contract():
    c = CONFIGS
    assert list(c) == ["c1_cpu_ref", "c2_decode", "c3_small_batch", "c4_prefill", "c5_mlp70b"]
    assert c["c1_cpu_ref"].bytes_algorithmic == 4_458_496
    assert c["c2_decode"].bytes_algorithmic == 11_478_528 and c["c2_decode"].groups == 86
    assert c["c3_small_batch"].bytes_algorithmic == 17_367_040
    assert c["c4_prefill"].flops == 481_036_337_152 and c["c4_prefill"].groups == 112
    assert c["c5_mlp70b"].flops == 962_072_674_304 and c["c5_mlp70b"].groups == 224


def test_infer_layout():
    x = torch.zeros(4, 64, dtype=torch.float16)
    assert infer_layout(x, torch.zeros(32, 16, dtype=torch.uint8), torch.zeros(1, 256, 4, dtype=torch.float16)) == "bl"
    assert infer_layout(x, torch.zeros(32, 8, dtype=torch.int16), torch.zeros(4096, 8, dtype=torch.float16)) == "bl"
    assert infer_layout(x, torch.zeros(64, 16, dtype=torch.uint8), torch.zeros(4, 256, 2, dtype=torch.float16)) == "ref"
    with pytest.raises(RuntimeError, match="neither"):
        infer_layout(x, torch.zeros(32, 15, dtype=torch.uint8), torch.zeros(1, 256, 4, dtype=torch.float16))
    # K = 2 * (columns of w) and K rows: both readings fit
    x2 = torch.zeros(4, 16, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="both"):
        infer_layout(x2, torch.zeros(16, 8, dtype=torch.uint8), torch.zeros(2, 256, 2, dtype=torch.float16))


def test_shard_inputs_are_slices_of_nothing_but_consistent():
    s = CONFIGS["c2_decode"]
    x0, idx0, cb0 = make_inputs(s, seed=3, n_rows=256, row0=0)
    x1, idx1, cb1 = make_inputs(s, seed=3, n_rows=256, row0=256)
    assert torch.equal(x0, x1)                       # X is replicated
    assert not torch.equal(idx0, idx1)               # shards differ
    assert idx0.shape == (256, 1024) and cb0.shape == (2, 256, 4)
    xa, ia, ca = make_inputs(s, seed=3, n_rows=256, row0=0)
    assert torch.equal(ia, idx0) and torch.equal(ca, cb0)  # deterministic
