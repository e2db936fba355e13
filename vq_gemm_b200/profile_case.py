"""Runs one benchmark configuration a few times on cuda:0 -- the command to put under a profiler.

    python -m vq_gemm_b200.profile_case c2_decode 8            # configuration, launches [, path]
    python -m vq_gemm_b200.profile_case c4_prefill 4 tensor_ts
    ncu --set full --clock-control none -k regex:vq_decode -s 5 -c 2 -o out python -m vq_gemm_b200.profile_case c2_decode 8
"""
import sys

import torch

import vq_gemm_b200 as V
from vq_gemm_b200.formats import CONFIGS, make_inputs


def main(argv):
    name = argv[0] if argv else "c2_decode"
    n = int(argv[1]) if len(argv) > 1 else 8
    path = argv[2] if len(argv) > 2 else "auto"
    s = CONFIGS[name]
    x, idx, cb = make_inputs(s, seed=0, device="cuda")
    y = None
    for _ in range(n):
        y = V.vq_gemm(x, idx, cb, rows_per_codebook=s.rows_per_codebook, layout="bl", path=path)
    torch.cuda.synchronize()
    if V.device_status() != 0:
        raise SystemExit("device status word set")
    print("ok", name, path, float(y.float().abs().mean()))


if __name__ == "__main__":
    main(sys.argv[1:])
