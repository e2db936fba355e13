"""The registered operator and the nn.Module on top of it."""
import pytest
import torch

import vq_gemm_b200 as V
from oracle import vq_oracle as O
from tests._util import assert_within_tolerance, bits
from vq_gemm_b200.linear import VQLinear

pytestmark = pytest.mark.gpu


def _layer(M=8, K=512, N=256, v=8, rpc=128, bias=False, seed=1):
    x, idx, cb = O.make_bl_inputs(M, K, N, v, 256, rpc, seed=seed)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(seed)) * 0.1).half() if bias else None
    return x, idx, cb, b, VQLinear(idx, cb, rpc, b).cuda()


def test_module_equals_the_functional_call_and_the_oracle():
    x, idx, cb, _, layer = _layer()
    y = layer(x.cuda())
    assert torch.equal(bits(y), bits(V.vq_gemm(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=128, layout="bl")))
    assert_within_tolerance(y.cpu(), O.vq_gemm_bl(x, idx, cb, 128))
    assert "in_features=512" in repr(layer)


def test_leading_dimensions_bias_and_state_dict():
    x, idx, cb, b, layer = _layer(M=12, bias=True)
    x3 = x.reshape(3, 4, -1).cuda()
    y = layer(x3)
    assert y.shape == (3, 4, 256)
    ref = O.vq_gemm_bl(x, idx, cb, 128).float() + b.float()
    assert_within_tolerance(y.reshape(12, 256).cpu(), ref.half())
    clone = VQLinear(torch.zeros_like(idx), torch.zeros_like(cb), 128, torch.zeros_like(b)).cuda()
    clone.load_state_dict(layer.state_dict())
    assert torch.equal(bits(clone(x3)), bits(y))
    assert torch.equal(layer.dequantized_weight().cpu(), O.dequant_bl_layout(idx, cb, 128))


def test_cuda_graph_capture_and_replay():
    x, idx, cb, _, layer = _layer(M=4, K=8192, N=512)      # K > 4096: the split-K counters are in play
    xs = x.cuda()
    eager = layer(xs).clone()
    static_x = xs.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(static_x)                                     # warm-up on the capture stream
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = layer(static_x)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(bits(out), bits(eager))
    static_x.copy_(xs * 2)
    g.replay()
    torch.cuda.synchronize()
    assert_within_tolerance(out.cpu(), O.vq_gemm_bl((x.float() * 2).half(), idx, cb, 128))
    assert V.device_status() == 0


def test_traceable_operator():
    x, idx, cb, _, layer = _layer()
    torch.library.opcheck(torch.ops.vq_gemm_b200.vq_linear.default, (x.cuda(), idx.cuda(), cb.cuda(), 128),
                          test_utils=("test_schema", "test_faketensor"))
    compiled = torch.compile(layer, backend="eager", fullgraph=True)
    assert torch.equal(bits(compiled(x.cuda())), bits(layer(x.cuda())))


def test_from_weight_quantises_and_runs():
    w = (torch.randn(256, 512, generator=torch.Generator().manual_seed(2)) * 0.05).half().cuda()
    layer = VQLinear.from_weight(w, v=8, entries=256, rows_per_codebook=128, iters=3)
    x = torch.randn(16, 512, generator=torch.Generator().manual_seed(3)).half().cuda()
    y = layer(x)
    dense = x.float() @ w.float().t()
    rel = float((y.float() - dense).norm() / dense.norm())
    assert rel < 0.7          # 1 bit per weight on Gaussian noise: coarse, but far from random indices (~1.4)
    rel_q = float((y.float() - x.float() @ layer.dequantized_weight().float().t()).abs().max())
    assert rel_q <= 2e-2 * (float(dense.abs().max()) + 1)


def test_residual_module_equals_the_functional_call_and_the_oracle():
    x, idx, cb = O.make_residual_inputs(24, 512, 256, 8, 256, 128, 2, seed=9)
    layer = VQLinear(idx, cb, 128).cuda()
    assert layer.residual and (layer.in_features, layer.out_features, layer.v) == (512, 256, 8)
    y = layer(x.reshape(2, 12, 512).cuda())
    assert y.shape == (2, 12, 256)
    assert torch.equal(bits(y.reshape(24, 256)), bits(V.vq_gemm_residual(x.cuda(), idx.cuda(), cb.cuda(), rows_per_codebook=128)))
    assert_within_tolerance(y.reshape(24, 256).cpu(), O.vq_gemm_bl_residual(x, idx, cb, 128))
    assert torch.equal(bits(layer.dequantized_weight()).cpu(), bits(O.dequant_bl_residual(idx, cb, 128)))
    torch.library.opcheck(torch.ops.vq_gemm_b200.vq_linear_residual.default, (x.cuda(), idx.cuda(), cb.cuda(), 128),
                          test_utils=("test_schema", "test_faketensor"))
    assert "stages=2" in repr(layer)
    assert V.device_status() == 0


def test_residual_quantiser_lowers_the_error_stage_by_stage():
    w = (torch.randn(256, 512, generator=torch.Generator().manual_seed(5)) * 0.05).half().cuda()
    errs = []
    for stages in (1, 2, 3):
        layer = VQLinear.from_weight(w, v=8, entries=256, rows_per_codebook=128, iters=4, stages=stages)
        assert layer.indices.shape == ((stages, 256, 64) if stages > 1 else (256, 64))
        errs.append(float((layer.dequantized_weight().float() - w.float()).norm() / w.float().norm()))
    assert errs[1] < 0.9 * errs[0] and errs[2] < 0.9 * errs[1]
    x = torch.randn(16, 512, generator=torch.Generator().manual_seed(6)).half().cuda()
    dense = x.float() @ w.float().t()
    y = layer(x)
    assert float((y.float() - dense).norm() / dense.norm()) < 1.3 * errs[2] + 1e-2
    # stage 0 of the residual quantiser is the plain quantiser with the same seed
    from vq_gemm_b200.quantize import kmeans_quantize, kmeans_quantize_residual
    i1, c1 = kmeans_quantize(w, v=8, entries=256, rows_per_codebook=128, iters=4, seed=0)
    i2, c2 = kmeans_quantize_residual(w, stages=2, v=8, entries=256, rows_per_codebook=128, iters=4, seed=0)
    assert torch.equal(i1, i2[0]) and torch.equal(bits(c1), bits(c2[0]))


def test_packed_module_equals_the_int16_layer():
    x, idx, cb = O.make_bl_inputs(40, 512, 256, 8, 4096, 0, seed=11, idx_dtype=torch.int16)
    layer = VQLinear(idx, cb, 0).cuda()
    packed = layer.pack()
    assert packed.packed and packed.indices.shape == (256, 96) and packed.in_features == 512
    y, yp = layer(x.cuda()), packed(x.reshape(2, 20, 512).cuda()).reshape(40, 256)
    assert_within_tolerance(yp.cpu(), O.vq_gemm_bl(x, idx, cb, 0))
    assert torch.equal(bits(packed.dequantized_weight()), bits(layer.dequantized_weight()))
    assert float((y.float() - yp.float()).abs().max()) <= 2e-2 * (float(y.abs().max()) + 1)
    torch.library.opcheck(torch.ops.vq_gemm_b200.vq_linear_packed12.default, (x.cuda(), packed.indices, cb.cuda(), 0),
                          test_utils=("test_schema", "test_faketensor"))
    assert set(packed.state_dict()) == {"indices", "codebook"} and "packed12=True" in repr(packed)


def test_gated_module_and_operator():
    from vq_gemm_b200.linear import VQGatedUp
    x, idx, cb = O.make_bl_inputs(160, 512, 512, 8, 256, 128, seed=7, cb_sigma=0.05)
    layer = VQGatedUp(idx, cb, 128).cuda()
    y = layer(x.reshape(4, 40, 512).cuda())
    assert y.shape == (4, 40, 256)
    assert_within_tolerance(y.reshape(160, 256).cpu(), O.vq_gemm_swiglu_bl(x, idx, cb, 128))
    torch.library.opcheck(torch.ops.vq_gemm_b200.vq_swiglu.default, (x.cuda(), idx.cuda(), cb.cuda(), 128),
                          test_utils=("test_schema", "test_faketensor"))
    gate = (torch.randn(128, 256, generator=torch.Generator().manual_seed(1)) * 0.05).half().cuda()
    up = (torch.randn(128, 256, generator=torch.Generator().manual_seed(2)) * 0.05).half().cuda()
    q = VQGatedUp.from_weights(gate, up, v=8, entries=256, rows_per_codebook=128, iters=2)
    xs = torch.randn(8, 256, generator=torch.Generator().manual_seed(3)).half().cuda()
    w = V.dequant(q.indices, q.codebook, rows_per_codebook=128).float()
    ref = torch.nn.functional.silu(xs.float() @ w[0::2].t()) * (xs.float() @ w[1::2].t())
    assert float((q(xs).float() - ref).abs().max()) <= 2e-2 * (float(ref.abs().max()) + 1)


def test_graph_with_layers_whose_scratch_grows_during_capture(monkeypatch):
    # the first layer is captured with a small scratch buffer, the second needs a much larger one: the small
    # one must stay alive (its address is baked into the graph) and keep its counters zero across replays
    from vq_gemm_b200 import ops
    monkeypatch.setattr(ops, "_MIN_WORKSPACE", 1 << 20)
    monkeypatch.setattr(ops, "_workspaces", {})      # torch hands out pooled streams: start without cached buffers
    monkeypatch.setattr(ops, "_retired", [])
    xa, ia, ca = O.make_bl_inputs(4, 8192, 512, 8, 256, 128, seed=31)        # split-K counters + partials
    xb, ib, cb = O.make_bl_inputs(300, 1024, 1280, 8, 256, 128, seed=32)     # prefill kernel: 37 MiB of partial tiles
    la, lb = VQLinear(ia, ca, 128).cuda(), VQLinear(ib, cb, 128).cuda()
    sa, sb = xa.cuda(), xb.cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            ya = la(sa)
            yb = lb(sb)
            ya2 = la(sa)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert V.device_status() == 0
    assert_within_tolerance(ya.cpu(), O.vq_gemm_bl(xa, ia, ca, 128))
    assert_within_tolerance(yb.cpu(), O.vq_gemm_bl(xb, ib, cb, 128))
    assert torch.equal(bits(ya2), bits(ya))
    assert len(ops._retired) >= 1
