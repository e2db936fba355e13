"""CPU restatement of the quantiser's rules (TEST INFRASTRUCTURE -- only tests may import this).

The reference has no quantiser (bench.py:83-85 draws random indices), so there is no reference
output to pin against: parity is against the rules stated in include/vqg.h, which are exact:

  assign   distance = sum_i (float32(w_i) - float32(c_i))^2, i ascending, each operation rounded to
           float32 separately; lowest index among equal distances
  update   exact integer sums of value * 2^24; mean = float32(float64(sum) * 2^-24 / count) -> fp16;
           entries with no member keep their value
  pack12   bytes [a & 255, (a >> 8) | ((b & 15) << 4), b >> 4] per pair (a, b)

numpy float32 arithmetic rounds every operation separately, which is exactly the rule.
"""
import numpy as np


def _groups(N, rows_per_codebook):
    rpc = N if (rows_per_codebook <= 0 or rows_per_codebook >= N) else rows_per_codebook
    return rpc, -(-N // rpc)


def assign(w: np.ndarray, cb: np.ndarray, rows_per_codebook: int = 0) -> np.ndarray:
    """w [N, K] float16, cb [G, C, v] float16 -> indices [N, K/v] (uint8 if C <= 256 else int16)."""
    N, K = w.shape
    G, C, v = cb.shape
    J = K // v
    rpc, groups = _groups(N, rows_per_codebook)
    out = np.empty((N, J), dtype=np.uint8 if C <= 256 else np.int16)
    for g in range(groups):
        r0, r1 = g * rpc, min(N, (g + 1) * rpc)
        x = w[r0:r1].astype(np.float32).reshape(-1, v)            # [S, v]
        e = cb[g].astype(np.float32)                               # [C, v]
        d = np.zeros((x.shape[0], C), dtype=np.float32)
        for i in range(v):                                          # ascending i, separate roundings
            t = x[:, i:i + 1] - e[None, :, i]
            d = d + t * t
        out[r0:r1] = np.argmin(d, axis=1).reshape(r1 - r0, J).astype(out.dtype)   # first minimum = lowest index
    return out


def update(w: np.ndarray, idx: np.ndarray, cb: np.ndarray, rows_per_codebook: int = 0) -> np.ndarray:
    """One Lloyd step; returns the new codebook [G, C, v] float16."""
    N, K = w.shape
    G, C, v = cb.shape
    rpc, groups = _groups(N, rows_per_codebook)
    new = cb.copy()
    for g in range(groups):
        r0, r1 = g * rpc, min(N, (g + 1) * rpc)
        fixed = np.round(w[r0:r1].astype(np.float64) * 16777216.0).astype(np.int64).reshape(-1, v)   # exact
        ids = idx[r0:r1].astype(np.int64).reshape(-1)
        ok = ids < C
        sums = np.zeros((C, v), dtype=np.int64)
        np.add.at(sums, ids[ok], fixed[ok])
        counts = np.bincount(ids[ok], minlength=C)
        has = counts > 0
        mean = (sums[has].astype(np.float64) * (1.0 / 16777216.0) / counts[has, None].astype(np.float64)).astype(np.float32)
        new[g][has] = mean.astype(np.float16)
    return new


def pack12(idx: np.ndarray) -> np.ndarray:
    a = idx.reshape(-1, 2).astype(np.uint32) & 0xFFF
    packed = a[:, 0] | (a[:, 1] << 12)
    out = np.stack([packed & 255, (packed >> 8) & 255, (packed >> 16) & 255], axis=1).astype(np.uint8)
    return out.reshape(*idx.shape[:-1], idx.shape[-1] * 3 // 2)


def unpack12(packed: np.ndarray) -> np.ndarray:
    p = packed.reshape(-1, 3).astype(np.uint32)
    word = p[:, 0] | (p[:, 1] << 8) | (p[:, 2] << 16)
    out = np.stack([word & 0xFFF, word >> 12], axis=1).astype(np.int16)
    return out.reshape(*packed.shape[:-1], packed.shape[-1] * 2 // 3)


def distortion(w: np.ndarray, idx: np.ndarray, cb: np.ndarray, rows_per_codebook: int = 0) -> float:
    """Mean squared error of the quantised weight, float64."""
    N, K = w.shape
    G, C, v = cb.shape
    rpc, groups = _groups(N, rows_per_codebook)
    err = 0.0
    for g in range(groups):
        r0, r1 = g * rpc, min(N, (g + 1) * rpc)
        deq = cb[g].astype(np.float64)[idx[r0:r1].astype(np.int64).reshape(-1)].reshape(r1 - r0, K)
        err += float(((w[r0:r1].astype(np.float64) - deq) ** 2).sum())
    return err / (N * K)
