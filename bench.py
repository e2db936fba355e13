#!/usr/bin/env python
"""Benchmark of the B200 VQ-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  A *step* is one product Y = X @ dequant(idx, codebook)^T on
the workload's synthetic inputs (seeded; X ~ N(0,1) fp16, codebook ~ N(0, 0.02) fp16, uniform
indices).  The default workload is the Llama-3-70B MLP up-projection shape (M=2048, K=8192,
N=28672, v=8, C=256, one codebook per 128 rows, 1 bit/weight): it fits one GPU and is the shape
that is N-sharded over 2/4/8 GPUs, so the same workload is timed at every N (strong scaling:
each rank owns N/G output columns and the fp16 output is assembled on every rank).

``value``      TFLOP/s (2*M*N*K per step) with inputs resident in HBM, CUDA events, max over ranks.
``e2e``        the same metric through the public Python entry point with HOST inputs: every step
               copies X, indices and codebooks from pinned host memory, runs the product and
               copies the rank's output columns back to pinned host memory.
``roofline``   the dominant kernel against the measured dense 16-bit tensor peak (or HBM peak for
               the M <= 16 workloads), from CUDA-event time of the kernel alone.
``shapes``     (N=1 only) the other single-GPU configurations, each with its own roofline, and
               cuBLAS fp16 (torch.matmul) on pre-dequantised weights for the prefill shapes.
``mlp70b``     (every N) the whole tensor-parallel MLP: gated up half N-sharded without a gather, down half
               K-sharded with the fused reduce-scatter; max over ranks.
``gated_mlp_up`` (N=1 only) SiLU(X g) * (X u) fused into the GEMM epilogue on the 70B gate+up shape.
``quantizer``  (N=1 only) the step before the product on a C4-sized layer: nearest-entry search
               against the fp32 pipe, one exact k-means update, 12-bit pack/unpack against HBM.
``cpu_baseline`` the torch CPU oracle (gather + fp32-accumulated matmul) on a bounded sample.
``sustained``  (N=1 only) the headline kernel launched back to back for at least two seconds with the clocks
               sampled: TFLOP/s against the sustained dense 16-bit peak, median SM clock, time x clock.
``cublas``     (N=1 only) cuBLAS fp16 (torch.matmul) on pre-dequantised weights for the two prefill shapes,
               fp32 and fp16 accumulation, in alternating blocks with this library's kernel.
``reference_cuda_kernels`` (N=1 only, when oracle/_ref holds them) the reference's own CUDA kernels rebuilt
               for sm_100a, on data in the reference's format, and this library on the same data.
The line ends with the compact records (``dequant``: the dequantisation kernels against the measured HBM bandwidth;
``shapes``: the per-configuration table); long per-kernel detail is under ``detail``.

``--profile-case NAME --launches n [--path p]`` runs n launches of one configuration and exits: the command to
put under a profiler (p: a product route, or ``dequant`` / ``dequant_ref`` / ``e2e_ref`` for the dequantisation kernels
and the product on data in the reference's format).

``--impl reference`` times the reference's torch path restated for CPU (oracle/vq_oracle.py) on
the host cores, same metric and workload, bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


def _traffic(kernel: str, workload: str):
    """DRAM bytes per launch of a kernel on a workload from the tracked record of ncu captures
    (dram__bytes_read.sum + dram__bytes_write.sum of one launch); None if there is no entry."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    try:
        for ln in open(path):
            f = ln.split()
            if len(f) >= 4 and not ln.startswith("#") and f[0] == kernel and f[1] == workload:
                return {"bytes": float(f[2]), "source": f"profiles/dram_traffic.txt (ncu capture at commit {f[3]})"}
    except OSError:
        pass
    return None


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU while a region runs: NVML read-only queries from a
    thread of this process every millisecond (the timed regions are a few milliseconds long), nvidia-smi polling
    every 100 ms where NVML's Python binding is missing."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    BITS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, index: int, enabled: bool = True, period_s: float = 0.001):
        self.index, self.rows, self.proc, self.enabled, self.period_s = index, [], None, enabled, period_s
        self.stop, self.t, self.source = threading.Event(), None, None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:   # the CUDA device's own PCI address: CUDA_VISIBLE_DEVICES may renumber the GPUs
            pr = torch.cuda.get_device_properties(self.index)
            bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
            return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll_nvml(self, nv, h):
        mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop.is_set():
            try:
                clk = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                mask = int(reasons_fn(h))
                self.rows.append([clk, mx, pw] + ["Active" if mask & bit else "Not Active" for _, bit in
                                                  (self.BITS[1], self.BITS[3], self.BITS[2], self.BITS[0])])
            except Exception:
                pass
            time.sleep(self.period_s)

    def __enter__(self):
        if not self.enabled:   # one sampler per job: the driver queries of eight pollers delay kernel launches
            return self
        try:
            nv, h = self._nvml_handle()
            self.t = threading.Thread(target=self._poll_nvml, args=(nv, h), daemon=True)
            self.t.start()
            self.source = f"nvml, {self.period_s * 1e3:g} ms"
            return self
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            self.source = "nvidia-smi, 100 ms"
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        self.stop.set()
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        elif self.t is not None:
            self.t.join(timeout=1)

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                clk, mxc, pw = float(r[0]), float(r[1]), float(r[2])
            except Exception:
                continue
            mx = max(mx, mxc)
            if pw > 250.0 or clk > 1000.0:  # under load (the power reading lags a region of a few milliseconds)
                sm.append(clk)
                for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                    if str(flag).lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples_under_load": len(sm), "source": self.source}


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _time_loop(fn, steps, warmup, barrier=None, counter=None):
    """W untimed steps, then exactly `steps` steps between a barrier + synchronize on both sides,
    timed with CUDA events on the launching stream.  Returns ms per step (and, with `counter`,
    the number of library kernel launches inside the timed region)."""
    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    c0 = counter() if counter else 0
    e0, e1 = _events()
    e0.record()
    t0 = time.perf_counter()
    for i in range(steps):
        fn()
    _time_loop.host_issue_ms = (time.perf_counter() - t0) * 1e3 / steps   # host time to enqueue one step
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    ms = e0.elapsed_time(e1) / steps
    return (ms, counter() - c0) if counter else ms


def _lookup_floor_us(shape, sm_mhz=1965.0, sms=148):
    """Time the shared-memory lookups alone would take: one 2v-byte codebook read per index at 128 bytes per
    clock and SM, conflict-free (the secondary roofline of the M <= 16 configurations)."""
    lookups = shape.N * (shape.K // shape.v)
    return lookups * 2.0 * shape.v / 128.0 / sms / sm_mhz


def _single_shape(V, shape, peaks, steps, warmup, alternatives=True):
    """One single-GPU configuration: kernel time over a ring of index buffers larger than L2.  Returns the
    compact entry for the table at the end of the line and the per-path detail."""
    from vq_gemm_b200.formats import make_inputs
    x, idx, cb = make_inputs(shape, seed=0, device="cuda")
    ring = 1
    if shape.bound == "hbm":
        ring = max(2, int(400e6 // shape.bytes_idx) + 1)
    idxs = [idx] + [idx.clone() for _ in range(ring - 1)]
    out = torch.empty((shape.M, shape.N), dtype=torch.float16, device="cuda")
    state = {"i": 0}

    def step():
        V.vq_gemm(x, idxs[state["i"] % ring], cb, rows_per_codebook=shape.rows_per_codebook, layout="bl", out=out)
        state["i"] += 1

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    # CUDA-graph replay of `ring` launches removes host launch gaps for the microsecond kernels
    def graph_ms(path, bufs=None, index_bits=None):
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        bufs = idxs if bufs is None else bufs
        with torch.cuda.stream(side):
            with torch.cuda.graph(g):
                for i in range(ring):
                    V.vq_gemm(x, bufs[i], cb, rows_per_codebook=shape.rows_per_codebook, layout="bl", path=path, out=out,
                              index_bits=index_bits)
        torch.cuda.current_stream().wait_stream(side)
        reps = max(3, steps // ring)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (reps * ring)

    ms = graph_ms("auto")
    e0, e1 = _events()
    compact = {"workload": shape.name, "M": shape.M, "K": shape.K, "N": shape.N, "us": round(ms * 1e3, 3)}
    detail = {"workload": shape.name, "v": shape.v, "C": shape.C, "ring_buffers": ring,
              "timing": "cuda-graph replay, CUDA events", "path": _path_name(V, shape)}
    if shape.bound == "hbm":
        a = shape.bytes_algorithmic / ms / 1e6
        compact.update({"gbs": round(a, 1), "bound": "hbm", "frac": round(a / peaks["hbm_gbs"], 4),
                        "frac_of_8000": round(a / 8000.0, 4), "bytes": shape.bytes_algorithmic,
                        "lookup_floor_us": round(_lookup_floor_us(shape), 2)})
        # both small-batch kernels, whichever the library picks by itself for this shape
        for alt in (("decode", "small_ts") if alternatives else ()):
            try:
                V.vq_gemm(x, idx, cb, rows_per_codebook=shape.rows_per_codebook, layout="bl", path=alt, out=out)
            except RuntimeError:
                continue
            ams = graph_ms(alt)
            detail["path_" + alt] = {"us": ams * 1e3, "gbs_compressed": shape.bytes_algorithmic / ams / 1e6}
        # 12-bit indices stored packed (1.5 bytes each) instead of in uint16: the same product from 25 % fewer index bytes
        if alternatives and shape.idx_bytes == 2 and shape.C <= 4096 and shape.v == 8:
            try:
                packed = [V.quantize.pack12(b) for b in idxs]
                V.vq_gemm(x, packed[0], cb, rows_per_codebook=shape.rows_per_codebook, out=out, index_bits=12)
                ams = graph_ms("auto", packed, 12)
                pbytes = shape.bytes_algorithmic - shape.bytes_idx // 4
                detail["packed12"] = {"us": ams * 1e3, "bytes": pbytes, "gbs_compressed": pbytes / ams / 1e6,
                                      "path": V.auto_path(shape.M, shape.N, shape.K, shape.v, shape.C, 12, shape.rows_per_codebook)}
                del packed
            except RuntimeError as e:
                detail["packed12"] = {"error": repr(e)}
    else:
        a = shape.flops / ms / 1e9
        compact.update({"tflops": round(a, 1), "bound": "tensor", "frac": round(a / peaks["tflops"], 4),
                        "frac_of_2250": round(a / 2250.0, 4)})
        # the other routes through the library: single-CTA fused kernel, and dequantise-then-dense
        for alt in (("tensor", "tensor_pair", "two_phase") if alternatives else ()):
            for _ in range(3):
                V.vq_gemm(x, idx, cb, rows_per_codebook=shape.rows_per_codebook, layout="bl", path=alt, out=out)
            torch.cuda.synchronize()
            n = max(5, min(steps, 30))
            e0.record()
            for _ in range(n):
                V.vq_gemm(x, idx, cb, rows_per_codebook=shape.rows_per_codebook, layout="bl", path=alt, out=out)
            e1.record()
            torch.cuda.synchronize()
            ams = e0.elapsed_time(e1) / n
            detail["path_" + alt] = {"tflops": shape.flops / ams / 1e9, "us": ams * 1e3}
    return compact, detail


def _path_name(V, shape):
    from vq_gemm_b200 import _lib
    code = _lib.load().vqg_auto_path(shape.M, shape.N, shape.K, shape.v, shape.C, shape.idx_bytes, shape.rows_per_codebook, 0)
    return {v: k for k, v in _lib.PATHS.items()}.get(code, str(code))


def _cublas_compare(V, shape, x=None, idx=None, cb=None):
    """cuBLAS fp16 on pre-dequantised weights (the reference's ref_gemm comparator, ref_gemm/cublas_gemm_fp16.cu:36-46)
    against this library's fused kernel, in alternating blocks of equal length so that all see the same clocks
    under the power cap.  Two cuBLAS accumulate modes: fp32 (like ours) and fp16 (CUBLAS_COMPUTE_16F, what the
    reference's wrapper asks for).  Dequantisation time is not charged to cuBLAS."""
    from vq_gemm_b200.formats import make_inputs
    if x is None:
        x, idx, cb = make_inputs(shape, seed=0, device="cuda")
    rpc = shape.rows_per_codebook
    out = torch.empty((shape.M, shape.N), dtype=torch.float16, device=x.device)
    w = V.dequant(idx, cb, rows_per_codebook=rpc)
    wt = w.t()
    ref = torch.empty((shape.M, shape.N), dtype=torch.float16, device=x.device)
    e0, e1 = _events()
    has16 = hasattr(torch.backends.cuda.matmul, "allow_fp16_accumulation")

    def ours():
        V.vq_gemm(x, idx, cb, rows_per_codebook=rpc, layout="bl", out=out)

    def cublas32():
        torch.matmul(x, wt, out=ref)

    def cublas16():
        torch.backends.cuda.matmul.allow_fp16_accumulation = True
        try:
            torch.matmul(x, wt, out=ref)
        finally:
            torch.backends.cuda.matmul.allow_fp16_accumulation = False

    def block(fn, n=20):
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    fns = [("ours", ours), ("cublas_acc32", cublas32)] + ([("cublas_acc16", cublas16)] if has16 else [])
    for _, fn in fns:
        block(fn, 5)
    t = {k: [] for k, _ in fns}
    for _ in range(5):
        for k, fn in fns:
            t[k].append(block(fn))
    med = {k: statistics.median(v) for k, v in t.items()}
    res = {"workload": shape.name, "blocks": 5, "launches_per_block": 20, "timing": "alternating blocks",
           "ours_us": round(med["ours"] * 1e3, 1), "ours_tflops": round(shape.flops / med["ours"] / 1e9, 1)}
    for k in ("cublas_acc32", "cublas_acc16"):
        if k in med:
            res[k] = {"us": round(med[k] * 1e3, 1), "tflops": round(shape.flops / med[k] / 1e9, 1),
                      "speedup_ours": round(med[k] / med["ours"], 3)}
    del w, wt, ref
    return res


def _sustained(V, shape, x, idx, cb, peaks, device_index, seconds=2.5):
    """The headline kernel launched back to back for `seconds` with the clocks sampled: the rate the chip
    sustains under its power cap, to set against the sustained dense 16-bit peak."""
    rpc = shape.rows_per_codebook
    out = torch.empty((shape.M, idx.shape[0]), dtype=torch.float16, device=x.device)
    e0, e1 = _events()
    for _ in range(5):
        V.vq_gemm(x, idx, cb, rows_per_codebook=rpc, layout="bl", out=out)
    torch.cuda.synchronize()
    n = 0
    with ClockSampler(device_index, period_s=0.02) as cs:
        t0 = time.perf_counter()
        e0.record()
        while time.perf_counter() - t0 < seconds:
            for _ in range(50):
                V.vq_gemm(x, idx, cb, rows_per_codebook=rpc, layout="bl", out=out)
            n += 50
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    c = cs.summary()
    tf = shape.flops / ms / 1e9
    return {"workload": shape.name, "launches": n, "seconds": round(ms * n / 1e3, 2), "us": round(ms * 1e3, 1),
            "tflops": round(tf, 1), "sm_mhz_median": c["sm_mhz"], "reasons": c["reasons"],
            "us_x_mhz": round(ms * 1e3 * c["sm_mhz"], 0) if c["sm_mhz"] else None,
            "frac_of_sustained_peak": round(tf / peaks["tflops_sustained"], 4) if peaks["tflops_sustained"] else None,
            "frac_of_burst_peak": round(tf / peaks["tflops"], 4)}


def _residual(V, peaks):
    """Residual (two-codebook) weights on the headline shape: 2 x 1 bit per weight, both stages looked up and added
    inside the prefill kernel."""
    import torch
    M, K, N, v, C, rpc, S = 2048, 8192, 28672, 8, 256, 128, 2
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, K, device="cuda", generator=g).half()
    idx = torch.randint(0, C, (S, N, K // v), device="cuda", generator=g, dtype=torch.int32).to(torch.uint8)
    cb = torch.stack([(torch.randn(N // rpc, C, v, device="cuda", generator=g) * (0.02 / 2 ** s)).half() for s in range(S)])
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    e0, e1 = _events()
    for _ in range(3):
        V.vq_gemm_residual(x, idx, cb, rows_per_codebook=rpc, out=out)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(10):
        V.vq_gemm_residual(x, idx, cb, rows_per_codebook=rpc, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    tf = 2.0 * M * N * K / ms / 1e9
    return {"workload": "c5 shape, residual weights (2 stages x 1 bit/weight)", "M": M, "K": K, "N": N, "v": v, "C": C,
            "stages": S, "us": round(ms * 1e3, 1), "tflops": round(tf, 1), "frac": round(tf / peaks["tflops"], 4)}


def _dequant_rates(V, peaks):
    """The bit-exact dequantisation kernels against the HBM roofline: algorithmic bytes (indices + codebooks + the
    fp16 weights written) per second, launches back to back over a ring of outputs larger than L2 (so that every
    launch also pays for the write-back of the one before it)."""
    rows = []

    def timed(call, ring):
        for i in range(2 * ring):
            call(i)
        e0, e1 = _events()
        torch.cuda.synchronize()
        n = 4 * ring
        e0.record()
        for i in range(n):
            call(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    g = torch.Generator(device="cuda").manual_seed(0)
    for name, (N, K, v, C, rpc, S, dt) in {
            "c5 weights": (28672, 8192, 8, 256, 128, 1, torch.uint8),
            "c4 weights": (14336, 4096, 4, 256, 128, 1, torch.uint8),
            "c3 weights": (8192, 8192, 8, 4096, 0, 1, torch.int16),
            "c5 weights, 2 residual stages": (28672, 8192, 8, 256, 128, 2, torch.uint8)}.items():
        G = 1 if rpc == 0 else N // rpc
        idx = torch.randint(0, C, (S, N, K // v), device="cuda", generator=g, dtype=torch.int32).to(dt)
        cb = (torch.randn(S, G, C, v, device="cuda", generator=g) * 0.02).half()
        ring = max(2, int(600e6 // (N * K * 2)) + 1)
        outs = [torch.empty(N, K, dtype=torch.float16, device="cuda") for _ in range(ring)]
        idxs = [idx.clone() for _ in range(ring)]
        if S == 1:
            ms = timed(lambda i: V.dequant(idxs[i % ring][0], cb[0], rows_per_codebook=rpc, out=outs[i % ring]), ring)
        else:
            ms = timed(lambda i: V.dequant_residual(idxs[i % ring], cb, rows_per_codebook=rpc, out=outs[i % ring]), ring)
        b = idx.numel() * idx.element_size() + cb.numel() * 2 + N * K * 2
        rows.append({"what": name, "layout": "bl", "us": round(ms * 1e3, 1), "mb": round(b / 1e6, 1),
                     "gbs": round(b / ms / 1e6), "frac_of_hbm": round(b / ms / 1e6 / peaks["hbm_gbs"], 3)})
        del outs, idxs
    for K, Nq in ((4096, 7168), (8192, 14336)):
        w = torch.randint(0, 256, (K, Nq), device="cuda", generator=g, dtype=torch.int32).to(torch.uint8)
        cb = (torch.randn(Nq // 4, 256, 2, device="cuda", generator=g) * 0.02).half()
        ring = max(2, int(600e6 // (K * Nq * 4)) + 1)
        outs = [torch.empty(K, 2 * Nq, dtype=torch.float16, device="cuda") for _ in range(ring)]
        ws = [w.clone() for _ in range(ring)]
        ms = timed(lambda i: V.dequant(ws[i % ring], cb, layout="ref", out=outs[i % ring]), ring)
        b = w.numel() + cb.numel() * 2 + K * Nq * 4
        rows.append({"what": f"reference format K={K} Nq={Nq}", "layout": "ref", "us": round(ms * 1e3, 1), "mb": round(b / 1e6, 1),
                     "gbs": round(b / ms / 1e6), "frac_of_hbm": round(b / ms / 1e6 / peaks["hbm_gbs"], 3)})
        del outs, ws
    return rows


def _quantizer(peaks, clocks_mhz):
    """Quantiser kernels on a layer of C4's size (N=14336, K=4096, v=4, 256 entries per 128 rows)."""
    from vq_gemm_b200 import quantize as VQ
    N, K, v, C, rpc = 14336, 4096, 4, 256, 128
    w = (torch.randn(N, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0)) * 0.02).half()
    cb = VQ.initial_codebook(w, v, C, rpc, seed=0)
    idx = VQ.assign(w, cb, rpc)
    e0, e1 = _events()

    def timed(fn, n=5):
        fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    t_assign = timed(lambda: VQ.assign(w, cb, rpc, out=idx))
    t_update = timed(lambda: VQ.kmeans_update(w, idx, cb.clone(), rpc))
    # search: per (sub-vector, entry) pair v subtractions, v multiplications, v additions, none fused
    lane_ops = 3.0 * v * C * (N * K / v)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    # two fp32 operations per lane and cycle: packed .f32x2 instructions, still one rounding per operation (no FMA by rule)
    fp32_peak = sms * 128 * 2 * clocks_mhz * 1e6
    idx12 = torch.randint(0, 4096, (8192, 8192), device="cuda").to(torch.int16)
    packed = VQ.pack12(idx12)
    t_pack = timed(lambda: VQ.pack12(idx12))
    t_unpack = timed(lambda: VQ.unpack12(packed))
    pack_bytes = idx12.numel() * 2 + packed.numel()
    return {"layer": {"N": N, "K": K, "v": v, "C": C, "rows_per_codebook": rpc},
            "assign": {"ms": t_assign, "subvectors_per_s": (N * K / v) / t_assign * 1e3,
                       "roofline": {"bound": "fp32", "achieved": lane_ops / t_assign / 1e6, "peak": fp32_peak / 1e9,
                                    "unit": "Gop/s", "frac": lane_ops / (t_assign * 1e-3) / fp32_peak,
                                    "peak_source": "SMs x 128 lanes x 2 (packed f32x2) x max SM clock; unfused sub/mul/add by the parity rule"}},
            "kmeans_update": {"ms": t_update, "gbs": (N * K * 2 + N * K / v) / t_update / 1e6,
                              "frac_of_hbm": (N * K * 2 + N * K / v) / t_update / 1e6 / peaks["hbm_gbs"]},
            "pack12": {"ms": t_pack, "gbs": pack_bytes / t_pack / 1e6, "frac_of_hbm": pack_bytes / t_pack / 1e6 / peaks["hbm_gbs"]},
            "unpack12": {"ms": t_unpack, "gbs": pack_bytes / t_unpack / 1e6,
                         "frac_of_hbm": pack_bytes / t_unpack / 1e6 / peaks["hbm_gbs"]}}


def _gated(V, peaks):
    """First half of a Llama-3-70B MLP on C5's shape: gate and up projections (2 x 28672 rows, interleaved)
    with SiLU(g) * u fused into the GEMM epilogue, against the product followed by an elementwise pass."""
    from vq_gemm_b200.formats import VQShape, make_inputs
    shape = VQShape("mlp70b_gate_up", 2048, 8192, 57344, 8, 256, 128, 1, "tensor")
    x, idx, cb = make_inputs(shape, seed=0, device="cuda")
    out = torch.empty((shape.M, shape.N // 2), dtype=torch.float16, device="cuda")
    full = torch.empty((shape.M, shape.N), dtype=torch.float16, device="cuda")
    e0, e1 = _events()

    def fused():
        V.vq_gemm_swiglu(x, idx, cb, rows_per_codebook=128, out=out)

    def unfused():
        V.vq_gemm(x, idx, cb, rows_per_codebook=128, layout="bl", out=full)
        torch.mul(torch.nn.functional.silu(full[:, 0::2]), full[:, 1::2], out=out)

    def block(fn, n=10):
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    for fn in (fused, unfused):
        block(fn, 3)
    tf, tu = [], []
    for _ in range(3):
        tf.append(block(fused))
        tu.append(block(unfused))
    f_ms, u_ms = statistics.median(tf), statistics.median(tu)
    return {"workload": shape.name, "M": shape.M, "K": shape.K, "N_out": shape.N // 2, "v": 8, "C": 256,
            "fused_ms": f_ms, "tflops": shape.flops / f_ms / 1e9, "frac_of_measured_peak": shape.flops / f_ms / 1e9 / peaks["tflops"],
            "product_then_elementwise_ms": u_ms, "speedup": u_ms / f_ms, "timing": "alternating blocks of 10"}


def _mlp(V, world, rank, dev, steps, warmup, barrier, reduce_max):
    """Tensor-parallel Llama-3-70B MLP on M = 2048 tokens, all of it compressed (1 bit per weight): the gated
    up half N-sharded (each rank keeps its slice of the activation, nothing is gathered) and the down half
    K-sharded with the fused reduce-scatter.  Every rank ends with its [M, 8192/G] block of the output."""
    from vq_gemm_b200.formats import VQShape, make_inputs
    from vq_gemm_b200.sharded import RowParallelVQGemm, shard_weights_k
    M, H, I = 2048, 8192, 28672
    up = VQShape("up", M, H, 2 * I, 8, 256, 128, 1, "tensor")
    down = VQShape("down", M, I, H, 8, 256, 128, 1, "tensor")
    n_up = 2 * I // world
    x, idx_u, cb_u = make_inputs(up, seed=1, device=dev, n_rows=n_up, row0=rank * n_up)
    _, idx_d_full, cb_d = make_inputs(down, seed=2, device=dev)
    idx_d = shard_weights_k(idx_d_full, world, rank)
    del idx_d_full
    act = torch.empty((M, n_up // 2), dtype=torch.float16, device=dev)
    rp = RowParallelVQGemm(M, H, device=dev)

    def step():
        V.vq_gemm_swiglu(x, idx_u, cb_u, rows_per_codebook=128, out=act)
        rp(act, idx_d, cb_d, 128)

    def up_only():
        V.vq_gemm_swiglu(x, idx_u, cb_u, rows_per_codebook=128, out=act)

    ms = reduce_max(_time_loop(step, steps, warmup, barrier))
    up_ms = reduce_max(_time_loop(up_only, max(5, steps // 2), 2, barrier))
    flops = 2.0 * M * H * 2 * I + 2.0 * M * I * H
    return {"workload": "llama3-70b MLP, M=2048, v=8, C=256: gated up (N-sharded, not gathered) + down (K-sharded, reduce-scatter)",
            "ms_per_step": ms, "tflops": flops / ms / 1e9, "up_ms": up_ms, "down_and_reduce_scatter_ms": ms - up_ms,
            "reduce_scatter_bytes_per_gpu": int(M * H * 2 * (world - 1) / world)}


def _reference_cuda_kernels(V):
    """Baseline leg (N=1, whenever oracle/_ref holds them): the reference's own CUDA kernels, rebuilt unmodified for
    sm_100a by oracle/build_ref.py, on data in the reference's format; and this library on the same data.
    The reference launchers print to stdout and (PROFILING 1) run 50 + 100 launches per call, so stdout is
    parked on /dev/null around them and the event time of one call is divided by 150."""
    import importlib.util
    from oracle import vq_oracle as O
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    launches = {"s1": 150, "s2_128": 150, "s2_512": 150, "s3_naive": 1, "s3_wasp": 150}
    out = []
    for tag, (M, K, Nq) in {"reference_default": (2048, 4096, 640), "c4_sized": (4096, 4096, 7168)}.items():
        x, w, cb = O.make_ref_inputs(M, K, Nq, seed=42)
        cb = (cb.float() * 0.02).half()
        xd, wd, cbd = x.cuda(), w.cuda(), cb.cuda()
        flops = 2.0 * M * K * Nq * 2
        e0, e1 = _events()
        for _ in range(3):
            ours = V.e2e_gemm(xd, wd, cbd)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            ours = V.e2e_gemm(xd, wd, cbd)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 20
        row = {"shape": tag, "M": M, "K": K, "Nq": Nq, "ours": {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1)}}
        for variant, per_call in launches.items():
            path = os.path.join(ref_dir, f"vq_gemm_cuda_{variant}.so")
            if not os.path.exists(path):
                row[variant] = {"unavailable": "not built (python oracle/build_ref.py)"}
                continue
            spec = importlib.util.spec_from_file_location(f"vq_gemm_cuda_{variant}", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            sys.stdout.flush()
            saved = os.dup(1)
            devnull = os.open(os.devnull, os.O_WRONLY)
            os.dup2(devnull, 1)
            try:
                calls = 1 if per_call > 1 else 20
                theirs = mod.e2e_gemm(xd, wd, cbd)          # warm-up call
                torch.cuda.synchronize()
                e0.record()
                for _ in range(calls):
                    theirs = mod.e2e_gemm(xd, wd, cbd)
                e1.record()
                torch.cuda.synchronize()
            finally:
                os.dup2(saved, 1)
                os.close(saved)
                os.close(devnull)
            rms = e0.elapsed_time(e1) / (calls * per_call)
            diff = float((theirs.float() - ours.float()).abs().max() / ours.float().abs().max())
            row[variant] = {"us": round(rms * 1e3, 1), "tflops": round(flops / rms / 1e9, 1),
                            "speedup_ours": round(rms / ms, 2), "rel_diff": round(diff, 4)}
        out.append(row)
    return out


def _use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU legs are meant to use every core
    this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))


def _cpu_sample(shape, seconds_budget=20.0):
    """Torch CPU oracle on a column block of the workload (full M and K)."""
    _use_all_host_threads()
    from oracle import vq_oracle as O
    from vq_gemm_b200.formats import make_inputs
    rpc = shape.rows_per_codebook
    n_rows = shape.N
    if rpc > 0:
        n_rows = min(shape.N, max(rpc, (shape.N // 8) // rpc * rpc))
    x, idx, cb = make_inputs(shape, seed=0, n_rows=n_rows if rpc > 0 else None)
    t0 = time.perf_counter()
    O.vq_gemm_bl(x, idx, cb, rpc)
    first = time.perf_counter() - t0
    iters = max(1, min(5, int(seconds_budget / max(first, 1e-3)) - 1))
    t0 = time.perf_counter()
    for _ in range(iters):
        O.vq_gemm_bl(x, idx, cb, rpc)
    dt = (time.perf_counter() - t0) / iters
    flops = 2.0 * shape.M * idx.shape[0] * shape.K
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "host_cpus": os.cpu_count(), "seconds_per_sample": dt,
            "sample": f"{idx.shape[0]} of {shape.N} output columns, full M={shape.M} and K={shape.K}; "
                      f"torch gather + fp32 matmul + fp16 cast, {iters} iterations"}


def run_reference(args, shape):
    """The reference's torch path on the host cores (CPU restatement): every step is the WHOLE product of the
    workload -- index gather into the codebooks, fp32-accumulated matmul, fp16 cast -- done in column blocks of whole
    codebook groups so that the dequantised weights of one block (not of the matrix) are alive at a time."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _use_all_host_threads()
    from oracle import vq_oracle as O
    from vq_gemm_b200.formats import make_inputs
    rpc = shape.rows_per_codebook
    x, idx, cb = make_inputs(shape, seed=0)
    nblk = 8 if (rpc > 0 and shape.N % (8 * rpc) == 0) else 1
    rows = shape.N // nblk

    def step():
        for b in range(nblk):
            if rpc > 0:
                O.vq_gemm_bl(x, idx[b * rows:(b + 1) * rows], cb[b * rows // rpc:(b + 1) * rows // rpc], rpc)
            else:
                O.vq_gemm_bl(x, idx[b * rows:(b + 1) * rows], cb, 0)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = shape.flops / dt / 1e12
    sample = f"all {shape.N} output columns per step (in {nblk} column blocks), full M and K"
    print(json.dumps({
        "impl": "reference", "metric": "vq_gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": shape.name, "M": shape.M, "K": shape.K, "N": shape.N, "v": shape.v, "C": shape.C,
                   "rows_per_codebook": rpc, "idx_bytes": shape.idx_bytes,
                   "note": "reference torch path (index gather + fp32-accumulated matmul) on host cores"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5_mlp70b")
    ap.add_argument("--mode", default="auto", choices=["auto", "peer", "multicast", "nccl"],
                    help="how the N-sharded output is assembled (auto: peer stores; both fused modes are timed after the headline for the record)")
    ap.add_argument("--lead-cols", type=int, default=0,
                    help="columns of a rank's block issued as a small first launch in the N-sharded mode (0: one launch per step)")
    ap.add_argument("--no-shapes", action="store_true", help="skip the per-configuration table")
    ap.add_argument("--no-mlp", action="store_true", help="skip the tensor-parallel MLP measurement")
    ap.add_argument("--no-baselines", action="store_true",
                    help="skip cuBLAS, the reference's own CUDA kernels (oracle/_ref) and the sustained leg")
    ap.add_argument("--profile-case", default=None, metavar="NAME",
                    help="run --launches launches of one configuration on cuda:0 and exit (for use under a profiler)")
    ap.add_argument("--launches", type=int, default=8)
    ap.add_argument("--path", default="auto")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from vq_gemm_b200.formats import CONFIGS, make_inputs
    if args.profile_case:
        import vq_gemm_b200 as V
        sc = CONFIGS[args.profile_case]
        x, idx, cb = make_inputs(sc, seed=0, device="cuda")
        y = None
        if args.path in ("dequant_ref", "e2e_ref"):
            # the configuration's M, K and N in the reference's own format: index matrix [K, N/2], a codebook per 8 outputs
            g = torch.Generator(device="cuda").manual_seed(0)
            w = torch.randint(0, 256, (sc.K, sc.N // 2), device="cuda", generator=g, dtype=torch.int32).to(torch.uint8)
            cbr = (torch.randn(sc.N // 8, 256, 2, device="cuda", generator=g) * 0.02).half()
        for _ in range(args.launches):
            if args.path == "dequant":
                y = V.dequant(idx, cb, rows_per_codebook=sc.rows_per_codebook)
            elif args.path == "dequant_ref":
                y = V.dequant(w, cbr, layout="ref")
            elif args.path == "e2e_ref":
                y = V.e2e_gemm(x, w, cbr)
            else:
                y = V.vq_gemm(x, idx, cb, rows_per_codebook=sc.rows_per_codebook, layout="bl", path=args.path)
        torch.cuda.synchronize()
        if V.device_status() != 0:
            raise SystemExit("device status word set")
        print("ok", args.profile_case, args.path, float(y.float().abs().mean()))
        return
    shape = CONFIGS[args.workload]
    if args.impl == "reference":
        run_reference(args, shape)
        return

    import torch.distributed as dist
    import vq_gemm_b200 as V
    from vq_gemm_b200.sharded import ShardedVQGemm, partition

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if world > 1 else None
    peaks = _peaks()

    rpc = shape.rows_per_codebook
    row0, n_local = partition(shape.N, world, rank, rpc)
    x_h, idx_h, cb_h = make_inputs(shape, seed=0, n_rows=n_local if rpc > 0 else None, row0=row0)
    x_h, idx_h, cb_h = x_h.pin_memory(), idx_h.pin_memory(), cb_h.pin_memory()
    x, idx, cb = x_h.to(dev), idx_h.to(dev), cb_h.to(dev)
    # How Y is assembled.  Every rank first finds out LOCALLY whether symmetric memory can be had at all, the
    # ranks agree on that (a rank that fails inside a collective constructor would leave the others waiting in
    # it), and only then build -- all in the same mode.  "auto": multimem stores through the switch where the
    # fabric has a multicast mapping, timed against plain peer stores, the faster one kept.
    def agree(flag_ok: bool) -> bool:
        if world == 1:
            return flag_ok
        t = torch.tensor([0 if flag_ok else 1], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t.item()) == 0

    mode = args.mode
    gather_modes = {}
    if world > 1 and mode != "nccl":
        try:
            import torch.distributed._symmetric_memory as symm_mem
            probe = symm_mem.empty(1024, dtype=torch.float16, device=dev)
            local_ok = True
            del probe
        except Exception as e:  # noqa: BLE001
            local_ok = False
            print(f"rank {rank}: symmetric memory unavailable ({e!r})", file=sys.stderr)
        if not agree(local_ok):
            mode = "nccl"
    if world > 1 and mode in ("auto", "multicast"):
        from vq_gemm_b200.sharded import multicast_available
        has_mc = agree(multicast_available(dev))
        if mode == "multicast" and not has_mc:
            mode = "peer"
        if mode == "auto":
            # peer stores: the multimem route measured within 1 % of them on 2 GPUs and slower on 4 and 8 (both are
            # timed after the headline, below, for the record -- before it they would only warm the part up)
            mode = "peer"
    if world == 1 and mode == "auto":
        mode = "peer"
    op = ShardedVQGemm(shape.M, shape.N, mode=mode, device=dev, lead_cols=args.lead_cols)

    # clock warm-up: the SM clock idles at a few hundred MHz.  Kept short: half a second of dense GEMMs already
    # runs the part into its power cap, and the configurations measured next are quoted at burst clocks.
    a = torch.randn(4096, 4096, device=dev, dtype=torch.float16)
    t0 = time.time()
    while time.time() - t0 < 0.1:
        a @ a
    torch.cuda.synchronize()

    # The microsecond configurations are latency-bound: their time scales with the SM clock, which sits near its
    # maximum in a decode loop but stays low for a while after a power-capped GEMM phase.  They are therefore
    # measured first, before the long tensor-bound loops.
    solo = world == 1 and rank == 0
    shapes, detail = [], {}
    if solo and not args.no_shapes:
        detail["shapes"] = []
        for name in ("c1_cpu_ref", "c2_decode", "c3_small_batch"):
            try:
                compact, det = _single_shape(V, CONFIGS[name], peaks, max(args.steps, 200), args.warmup)
                shapes.append(compact)
                detail["shapes"].append(det)
            except Exception as e:  # keep the headline line even if a side measurement fails
                shapes.append({"workload": name, "error": repr(e)})
        # the dequantisation kernels, HBM-bound, before anything heats the part up
        try:
            detail["dequant"] = _dequant_rates(V, peaks)
        except Exception as e:
            detail["dequant"] = {"error": repr(e)}
        # C4 in a short burst as well (25 launches); its alternative routes are timed with the long extras below
        try:
            compact, _ = _single_shape(V, CONFIGS["c4_prefill"], peaks, 20, args.warmup, alternatives=False)
            shapes.append(compact)
        except Exception as e:
            shapes.append({"workload": "c4_prefill", "error": repr(e)})

    def step():
        op(x, idx, cb, rpc)

    with ClockSampler(local, enabled=(rank == 0)) as clocks:
        ms, launches = _time_loop(step, args.steps, args.warmup, barrier, counter=V.launch_count)
        host_issue_ms = _time_loop.host_issue_ms

        # kernel alone (no barriers, local columns only) for the roofline
        def kernel_only():
            V.vq_gemm(x, idx, cb, rows_per_codebook=rpc, layout="bl", out=kout)
        kout = torch.empty((shape.M, n_local), dtype=torch.float16, device=dev)
        # with one rank a step IS the kernel (no barriers, no peer copies): reuse its time rather than a
        # second loop that would run at a different point of the power/clock curve
        kms = ms if world == 1 else _time_loop(kernel_only, max(10, args.steps // 2), 3, None)

        # end to end: host inputs in, host output out, EVERY step -- as a serving loop would run it: three
        # streams (copy-in, compute, copy-out) over double-buffered device inputs and outputs, so step i+1's
        # input copy and step i-1's output copy overlap step i's kernel.  Every step still moves all of its
        # inputs (X, indices, codebooks) from pinned host memory and its output block back to pinned memory.
        # With G ranks on one host every rank copies only its M/G rows of X in and the ranks all-gather X over
        # NVLink (ShardedVQGemm.gather_x), so the host link carries X once per step, not G times.
        ops = [op, ShardedVQGemm(shape.M, shape.N, mode=mode, device=dev, lead_cols=args.lead_cols)]
        y_h = [torch.empty((shape.M, n_local), dtype=torch.float16).pin_memory() for _ in range(2)]
        ins = [(torch.empty_like(x), torch.empty_like(idx), torch.empty_like(cb)) for _ in range(2)]
        shard_x = world > 1 and shape.M % world == 0
        m_rows = shape.M // world if shard_x else shape.M
        xr_h = x_h[rank * m_rows:(rank + 1) * m_rows] if shard_x else x_h     # a view of the pinned X
        xr = [torch.empty((m_rows, shape.K), dtype=torch.float16, device=dev) for _ in range(2)]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        cur = torch.cuda.current_stream(dev)
        in_ready = [torch.cuda.Event() for _ in range(2)]
        comp_done = [torch.cuda.Event() for _ in range(2)]
        out_free = [torch.cuda.Event() for _ in range(2)]

        def e2e_run(n):
            start = torch.cuda.Event()
            start.record(cur)
            s_in.wait_event(start)
            s_out.wait_event(start)
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(comp_done[b])       # the kernel two steps back has read these buffers
                    (xr[b] if shard_x else ins[b][0]).copy_(xr_h, non_blocking=True)
                    ins[b][1].copy_(idx_h, non_blocking=True)
                    ins[b][2].copy_(cb_h, non_blocking=True)
                    in_ready[b].record(s_in)
                cur.wait_event(in_ready[b])
                if i >= 2:
                    cur.wait_event(out_free[b])             # its previous output has left the device
                if shard_x:
                    ops[b].gather_x(xr[b], out=ins[b][0])
                y = ops[b](ins[b][0], ins[b][1], ins[b][2], rpc)
                comp_done[b].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(comp_done[b])
                    y_h[b].copy_(y[:, row0:row0 + n_local], non_blocking=True)
                    out_free[b].record(s_out)
            for b in range(2):
                cur.wait_event(out_free[b])

        e2e_steps = args.steps
        e2e_run(4)
        if barrier:
            barrier()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        e2e_run(e2e_steps)
        e1.record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        ems = e0.elapsed_time(e1) / e2e_steps
    status = V.device_status()

    multi = None
    if world > 1:
        # both fused ways of assembling Y, 10 timed steps each after 3 warm-up steps, max over ranks (for the record:
        # the headline above ran in `mode`)
        if mode in ("peer", "multicast") and args.mode == "auto":
            try:
                from vq_gemm_b200.sharded import multicast_available
                cands = ["peer"] + (["multicast"] if agree(multicast_available(dev)) else [])
                for cand in cands:
                    trial = op if cand == mode else ShardedVQGemm(shape.M, shape.N, mode=cand, device=dev, lead_cols=args.lead_cols)
                    tms = _time_loop(lambda: trial(x, idx, cb, rpc), 10, 3, barrier)
                    tt = torch.tensor([tms], device=dev, dtype=torch.float64)
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                    gather_modes[cand] = float(tt.item())
                    del trial
            except Exception as e:  # noqa: BLE001
                gather_modes["error"] = repr(e)
        multi = {"gather_modes_trial_ms": gather_modes or None}
        # NVLink rate of this box: every rank reads 100 MB from its right neighbour's symmetric buffer at the same
        # time (plain copy-engine peer copy), max time over ranks
        try:
            hdl = op._hdl
            nelem = 50_000_000
            peer = hdl.get_buffer((rank + 1) % world, (nelem,), torch.float16, 0)
            dst = torch.empty(nelem, dtype=torch.float16, device=dev)
            for _ in range(2):
                dst.copy_(peer)
            torch.cuda.synchronize(); dist.barrier()
            e0, e1 = _events()
            e0.record()
            for _ in range(5):
                dst.copy_(peer)
            e1.record()
            torch.cuda.synchronize()
            tt = torch.tensor([e0.elapsed_time(e1) / 5], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            multi["link_gbs"] = nelem * 2 / float(tt.item()) / 1e6
            del dst, peer
        except Exception as e:  # noqa: BLE001
            multi["link_gbs"] = None
            multi["link_error"] = repr(e)
        # correctness of the gathered Y on every rank: bit for bit against the NCCL all-gather of the same blocks,
        # and this rank's own columns against the CPU oracle on a seeded 64 x 1028 subset
        try:
            from oracle import vq_oracle as O
            y_fused = op(x, idx, cb, rpc).clone()
            ref_op = ShardedVQGemm(shape.M, shape.N, mode="nccl", device=dev, lead_cols=args.lead_cols)
            y_nccl = ref_op(x, idx, cb, rpc)
            torch.cuda.synchronize()
            same = bool(torch.equal(y_fused.view(torch.int16), y_nccl.view(torch.int16)))
            g = torch.Generator().manual_seed(1 + rank)
            rows = torch.randperm(shape.M, generator=g)[:64].sort().values
            cols = torch.cat([torch.randperm(n_local, generator=g)[:1024], torch.tensor([0, 127, 128, n_local - 1])]).unique()
            sub = O.vq_gemm_bl_rows(x_h, idx_h, cb_h, rpc, rows, cols)
            got = y_fused[:, row0:row0 + n_local].cpu()[rows][:, cols]
            tol = O.check_tolerance(got, sub)["ok"]
            okt = torch.tensor([1 if (same and tol) else 0], device=dev)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            multi["gather_check"] = "bitwise+oracle ok" if int(okt.item()) == 1 else f"FAILED (rank {rank}: bitwise={same} oracle={tol})"
            del ref_op, y_nccl, y_fused
        except Exception as e:  # noqa: BLE001
            multi["gather_check"] = "error: " + repr(e)

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms, kms, ems = reduce_max(ms), reduce_max(kms), reduce_max(ems)
    h2d = xr_h.numel() * 2 + idx_h.numel() * idx_h.element_size() + cb_h.numel() * 2
    d2h = y_h[0].numel() * 2
    flops = shape.flops
    kflops = 2.0 * shape.M * n_local * shape.K
    tr = _traffic("vq_tensor_ts_kernel" if shape.bound == "tensor" else "vq_decode_kernel", shape.name) if world == 1 else None
    if shape.bound == "tensor":
        ach = kflops / kms / 1e9
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"],
                "traffic": tr["bytes"] if tr else None, "traffic_source": tr["source"] if tr else None,
                "traffic_algorithmic": shape.bytes_algorithmic if world == 1 else None,
                "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                "frac_of_sustained": ach / peaks["tflops_sustained"] if peaks["tflops_sustained"] else None,
                "frac_of_nominal_2250": ach / 2250.0, "kernel": "vq_tensor_ts_kernel", "kernel_us": kms * 1e3}
    else:
        b = shape.bytes_algorithmic / world
        ach = b / kms / 1e6
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                "traffic": tr["bytes"] if tr else None, "traffic_source": tr["source"] if tr else None,
                "peak_source": peaks["source"], "kernel": "vq_decode_kernel", "kernel_us": kms * 1e3}

    line = {
        "metric": "vq_gemm_tflops", "value": flops / ms / 1e9, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": shape.name, "M": shape.M, "K": shape.K, "N": shape.N, "v": shape.v, "C": shape.C,
                   "rows_per_codebook": rpc, "idx_bytes": shape.idx_bytes, "parallelism": f"N-sharded x{world}",
                   "gather": mode if world > 1 else "none",
                   "l2": "working set (indices + X + Y = 180 MB) larger than the 126 MB L2"},
        "e2e": {"value": flops / ems / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ems, "steps": e2e_steps,
                "pipeline": "3 streams, double-buffered; every step copies X" + (" (this rank's M/G rows, then all-gathered over NVLink)" if world > 1 else "")
                            + " + indices + codebooks in and its Y block out"},
        "gpu_launches": int(launches),
        "host_issue_ms_per_step": host_issue_ms,
        "roofline": roof,
        "clocks": clocks.summary(),
        "device_status": status,
    }
    if multi is not None:
        # what the link allows: every rank must RECEIVE (G-1)/G of Y while it computes its block
        ingress = shape.M * (shape.N - n_local) * 2
        multi["ingress_bytes_per_gpu"] = ingress
        if multi.get("link_gbs"):
            multi["ingress_ms_at_link"] = ingress / multi["link_gbs"] / 1e6
            multi["step_lower_bound_ms"] = max(kms, multi["ingress_ms_at_link"])
            multi["step_over_bound"] = ms / multi["step_lower_bound_ms"]
        multi["lead_cols"] = op._lead(rpc)      # columns issued as a small first launch (0: one launch per step)
        multi["kernel_alone_ms"] = kms
        multi["exposed_gather_ms"] = ms - kms
        line["multi_gpu"] = multi
    if not args.no_mlp:
        try:
            mlp = _mlp(V, world, rank, dev, args.steps, args.warmup, barrier, reduce_max)
        except Exception as e:
            mlp = {"error": repr(e)}
        line["mlp70b"] = mlp
    if solo and not args.no_shapes:
        try:
            _, det = _single_shape(V, CONFIGS["c4_prefill"], peaks, max(args.steps, 200), args.warmup)
            detail["shapes"].append(det)
        except Exception as e:
            detail["shapes"].append({"workload": "c4_prefill", "error": repr(e)})
        try:
            detail["gated_mlp_up"] = _gated(V, peaks)
        except Exception as e:
            detail["gated_mlp_up"] = {"error": repr(e)}
        try:
            detail["residual"] = _residual(V, peaks)
        except Exception as e:
            detail["residual"] = {"error": repr(e)}
        try:
            detail["quantizer"] = _quantizer(peaks, line["clocks"].get("sm_max_mhz") or 1965.0)
        except Exception as e:
            detail["quantizer"] = {"error": repr(e)}
    if detail:
        line["detail"] = detail
    if rank == 0 and world == 1:
        try:
            line["cpu_baseline"] = _cpu_sample(shape)
        except Exception as e:
            line["cpu_baseline"] = {"error": repr(e)}
    # the compact records the line ends with
    if solo and not args.no_baselines:
        if os.path.exists(os.path.join(ROOT, "oracle", "_ref", "vq_gemm_cuda_s1.so")):
            try:
                line["reference_cuda_kernels"] = _reference_cuda_kernels(V)
            except Exception as e:
                line["reference_cuda_kernels"] = {"error": repr(e)}
        else:
            line["reference_cuda_kernels"] = {"unavailable": "oracle/_ref not built (python oracle/build_ref.py)"}
        try:
            line["sustained"] = _sustained(V, shape, x, idx, cb, peaks, local)
        except Exception as e:
            line["sustained"] = {"error": repr(e)}
        cub = []
        for name in ("c4_prefill", "c5_mlp70b"):
            try:
                same = name == shape.name
                cub.append(_cublas_compare(V, CONFIGS[name], *((x, idx, cb) if same else ())))
            except Exception as e:
                cub.append({"workload": name, "error": repr(e)})
        line["cublas"] = cub
    if isinstance(detail.get("dequant"), list):
        # compact copy for the tail of the line: the dequantisation kernels against the measured HBM bandwidth
        line["dequant"] = [{"what": r["what"], "us": r["us"], "gbs": r["gbs"], "frac_of_hbm": r["frac_of_hbm"]}
                           for r in detail["dequant"]]
    if shapes:
        line["shapes"] = shapes
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
