"""Generates tests/golden/*.npz by running the REFERENCE's own oracle code on CPU.

Run it where the reference tree is checked out (its location is taken from VQG_REFERENCE_DIR):

    python tests/golden/make_golden.py

It imports the reference's ``bench.py`` (so ``vq_gemm_reference``, bench.py:37-57, is the
reference's code, not a restatement) with three stand-ins for things that cannot exist
on a CPU-only machine:

* ``matplotlib.pyplot`` -- absent from the image; never called by ``vq_gemm_reference``;
* the five ``vq_gemm_cuda_s*`` kernel modules -- empty stand-ins, never called;
* ``vq_gemm_cuda_cublas_gemm.gemm`` -- the cuBLAS fp16 product.  The stand-in records its
  second argument (the gathered weights ``w_decoded``, which is what these fixtures pin
  bit-exactly) and returns the fp32-accumulated product rounded to fp16.

The fixtures hold inputs, the reference's gathered weights and that product, for small
REF-layout cases.  One of them (``ref_nq4_bridge``, Nq = 4) is at the same time a BL-layout case:
with a single codebook the reference's gather equals the generalised rule with v = 2, so the
BL gather is checked against bytes the reference's code produced.  BL-layout cases (no reference implementation exists) are written by
the scalar-loop rule in oracle/vq_oracle.py so that later changes to the vectorised
oracle or to the kernels are caught.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("VQG_REFERENCE_DIR")


def import_reference_bench():
    if not REF or not os.path.isdir(REF):
        raise SystemExit("set VQG_REFERENCE_DIR to the reference checkout")
    captured = {}

    def gemm(inp, w):
        captured["w_decoded"] = w.clone()
        return (inp.float() @ w.float()).half()

    cublas = types.ModuleType("vq_gemm_cuda_cublas_gemm")
    cublas.gemm = gemm
    sys.modules["vq_gemm_cuda_cublas_gemm"] = cublas
    for name in ("s1", "s2_128", "s2_512", "s3_naive", "s3_wasp"):
        sys.modules[f"vq_gemm_cuda_{name}"] = types.ModuleType(f"vq_gemm_cuda_{name}")
    mpl = types.ModuleType("matplotlib")
    mpl.pyplot = types.ModuleType("matplotlib.pyplot")
    sys.modules["matplotlib"] = mpl
    sys.modules["matplotlib.pyplot"] = mpl.pyplot
    os.environ["KERNELS"] = "s1"            # bench.py:20-28 indexes a dict with it at import
    sys.path.insert(0, REF)
    bench = importlib.import_module("bench")
    assert os.path.dirname(os.path.abspath(bench.__file__)) == os.path.abspath(REF)
    return bench, captured


def main():
    sys.path.insert(0, ROOT)
    from oracle import vq_oracle as O

    only = set(sys.argv[1:])          # fixture names to (re)write; none given: all of them
    want = lambda tag: not only or tag in only
    bench = captured = None
    if not only or any(t.startswith("ref_") for t in only):
        bench, captured = import_reference_bench()

    # REF-layout cases: (M, K, Nq, seed)
    for tag, (M, K, Nq, seed) in {
        "ref_small": (128, 64, 64, 42),
        "ref_two_tiles": (256, 96, 128, 7),
        "ref_ragged": (5, 32, 8, 3),
        # Nq = 4: the reference's gather uses ONE codebook for all four index columns, so its w_decoded [K, 8]
        # is also what the generalised (BL) rule gives for idx = w read as [N = K rows, 4 indices], v = 2,
        # single codebook -- the one case in which the reference's own code pins the BL gather
        "ref_nq4_bridge": (16, 2048, 4, 11),
    }.items():
        if not want(tag):
            continue
        x, w, cb = O.make_ref_inputs(M, K, Nq, seed=seed)
        y = bench.vq_gemm_reference(x, w, cb)
        np.savez_compressed(
            os.path.join(HERE, f"{tag}.npz"),
            x=x.numpy(), w=w.numpy(), codebook=cb.numpy(),
            w_decoded=captured["w_decoded"].numpy(), y=y.numpy(),
            meta=np.array([M, K, Nq, seed]),
        )
        print(tag, "written", tuple(y.shape))

    # BL-layout cases: (M, K, N, v, C, rows_per_codebook, seed)
    for tag, (M, K, N, v, C, rpc, seed) in {
        "bl_v4_c256_groups": (3, 64, 256, 4, 256, 128, 0),
        "bl_v8_c4096_single": (16, 128, 48, 8, 4096, 0, 1),
        "bl_v8_c256_groups": (130, 128, 256, 8, 256, 128, 2),
    }.items():
        if not want(tag):
            continue
        x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=seed)
        wdec = O.dequant_bl_scalar(idx, cb, rpc)
        y = O.matmul_fp32acc(x, wdec)
        np.savez_compressed(
            os.path.join(HERE, f"{tag}.npz"),
            x=x.numpy(), idx=idx.numpy(), codebook=cb.numpy(),
            w_decoded=wdec.numpy(), y=y.numpy(),
            meta=np.array([M, K, N, v, C, rpc, seed]),
        )
        print(tag, "written", tuple(y.shape))


    # residual (two-codebook) case, written by the scalar-loop statement of the rule: (M, K, N, v, C, rpc, stages, seed)
    for tag, (M, K, N, v, C, rpc, stages, seed) in {"bl_residual_v8_c256_s2": (20, 128, 256, 8, 256, 128, 2, 3)}.items():
        if not want(tag):
            continue
        x, idx, cb = O.make_residual_inputs(M, K, N, v, C, rpc, stages=stages, seed=seed)
        wdec = O.dequant_bl_residual_scalar(idx, cb, rpc)
        y = O.matmul_fp32acc(x, wdec)
        np.savez_compressed(os.path.join(HERE, f"{tag}.npz"), x=x.numpy(), idx=idx.numpy(), codebook=cb.numpy(),
                            w_decoded=wdec.numpy(), y=y.numpy(), meta=np.array([M, K, N, v, C, rpc, stages, seed]))
        print(tag, "written", tuple(y.shape))

    # 12-bit indices packed two to three bytes (little end first): the packing written out byte by byte here,
    # the weights by the scalar-loop statement of the gather on the unpacked indices: (M, K, N, v, C, rpc, seed)
    for tag, (M, K, N, v, C, rpc, seed) in {"bl_v8_c4096_packed12": (12, 128, 64, 8, 4096, 0, 5)}.items():
        if not want(tag):
            continue
        x, idx, cb = O.make_bl_inputs(M, K, N, v, C, rpc, seed=seed, idx_dtype=torch.int16)
        flat = idx.numpy().astype(np.int64).reshape(N, -1)
        packed = np.zeros((N, flat.shape[1] * 3 // 2), dtype=np.uint8)
        for n in range(N):
            for j in range(0, flat.shape[1], 2):
                a, b = int(flat[n, j]), int(flat[n, j + 1])
                packed[n, 3 * (j // 2):3 * (j // 2) + 3] = [a & 255, (a >> 8) | ((b & 15) << 4), b >> 4]
        wdec = O.dequant_bl_scalar(idx, cb, rpc)
        y = O.matmul_fp32acc(x, wdec)
        np.savez_compressed(os.path.join(HERE, f"{tag}.npz"), x=x.numpy(), idx=idx.numpy(), packed=packed, codebook=cb.numpy(),
                            w_decoded=wdec.numpy(), y=y.numpy(), meta=np.array([M, K, N, v, C, rpc, seed]))
        print(tag, "written", tuple(y.shape))


if __name__ == "__main__":
    main()
