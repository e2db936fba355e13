"""Shape rule of the registered operator without a GPU (fake tensors), and module bookkeeping."""
import pytest
import torch

from vq_gemm_b200.linear import VQLinear


def test_fake_tensor_rule_gives_shape_and_dtype():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(5, 64, dtype=torch.float16, device="cuda")
        idx = torch.empty(32, 16, dtype=torch.uint8, device="cuda")
        cb = torch.empty(1, 256, 4, dtype=torch.float16, device="cuda")
        y = torch.ops.vq_gemm_b200.vq_linear(x, idx, cb, 0)
        assert y.shape == (5, 32) and y.dtype == torch.float16 and y.device.type == "cuda"
        with pytest.raises(RuntimeError):
            torch.ops.vq_gemm_b200.vq_linear(x, idx, torch.empty(1, 256, 8, dtype=torch.float16, device="cuda"), 0)


def test_fake_tensor_rule_of_the_residual_operator():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(5, 64, dtype=torch.float16, device="cuda")
        idx = torch.empty(2, 32, 16, dtype=torch.uint8, device="cuda")
        cb = torch.empty(2, 1, 256, 4, dtype=torch.float16, device="cuda")
        y = torch.ops.vq_gemm_b200.vq_linear_residual(x, idx, cb, 0)
        assert y.shape == (5, 32) and y.dtype == torch.float16
        with pytest.raises(RuntimeError):
            torch.ops.vq_gemm_b200.vq_linear_residual(x, idx, cb[:1], 0)


def test_residual_module_bookkeeping():
    idx = torch.zeros(2, 256, 64, dtype=torch.uint8)
    cb = torch.zeros(2, 2, 256, 8, dtype=torch.float16)
    layer = VQLinear(idx, cb, 128)
    assert layer.residual and (layer.in_features, layer.out_features, layer.v) == (512, 256, 8)
    with pytest.raises(ValueError):
        VQLinear(idx, cb[:1], 128)                 # one codebook array per stage
    with pytest.raises(ValueError):
        VQLinear(idx, cb[:, :1], 128)              # two groups of rows need two codebooks per stage
    with pytest.raises(ValueError):
        VQLinear(idx, cb[0], 128)


def test_packed_module_bookkeeping_and_fake_rule():
    from torch._subclasses.fake_tensor import FakeTensorMode
    pk = torch.zeros(64, 96, dtype=torch.uint8)              # 64 indices of 12 bits per row
    cb = torch.zeros(1, 4096, 8, dtype=torch.float16)
    layer = VQLinear(pk, cb, 0, index_bits=12)
    assert layer.packed and (layer.in_features, layer.out_features) == (512, 64)
    with pytest.raises(ValueError):
        VQLinear(torch.zeros(64, 95, dtype=torch.uint8), cb, 0, index_bits=12)
    with pytest.raises(ValueError):
        VQLinear(pk, cb, 0, index_bits=10)
    with FakeTensorMode():
        x = torch.empty(5, 512, dtype=torch.float16, device="cuda")
        y = torch.ops.vq_gemm_b200.vq_linear_packed12(x, torch.empty(64, 96, dtype=torch.uint8, device="cuda"),
                                                       torch.empty(1, 4096, 8, dtype=torch.float16, device="cuda"), 0)
        assert y.shape == (5, 64) and y.dtype == torch.float16


def test_module_bookkeeping_and_checks():
    idx = torch.zeros(256, 64, dtype=torch.uint8)
    cb = torch.zeros(2, 256, 8, dtype=torch.float16)
    layer = VQLinear(idx, cb, 128)
    assert (layer.in_features, layer.out_features, layer.v) == (512, 256, 8)
    assert set(layer.state_dict()) == {"indices", "codebook"}
    with pytest.raises(ValueError):
        VQLinear(idx, cb[:1], 128)                 # two groups of rows need two codebooks
    with pytest.raises(ValueError):
        VQLinear(idx.float(), cb, 128)
    with pytest.raises(RuntimeError, match="no CPU path|CUDA"):
        layer(torch.zeros(1, 512, dtype=torch.float16))


def test_no_cpu_fallback_for_the_operator():
    # the operator is registered for CUDA only: CPU tensors are refused by the dispatcher
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.vq_gemm_b200.vq_linear(torch.zeros(1, 8, dtype=torch.float16), torch.zeros(4, 2, dtype=torch.uint8),
                                         torch.zeros(1, 256, 4, dtype=torch.float16), 0)
