// Bit-exact dequantisation kernels (pure gathers; HBM-bound) and the shape-agnostic
// CUDA-core VQ-GEMM used for shapes none of the specialised kernels accept.
//
//   BL  : W[n, v*j + r]       = cb[n / rows_per_cb][ idx[n, j] ][r]   -> W    [N, K]
//   REF : Wdec[k, 2*n + r]    = cb[n / 4][ w[k, n] ][r]               -> Wdec [K, 2*Nq]
//         (reference strategy_1/src.cu:268-321 computes the same matrix)
//   REF transposed            : WdecT [2*Nq, K]  (K-major operand for the dense tensor kernel)
#include "common.cuh"

namespace vqg {

__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

template <int V> struct Entry;
template <> struct Entry<2> { using T = uint32_t; };
template <> struct Entry<4> { using T = uint2; };
template <> struct Entry<8> { using T = uint4; };

// One block = 16 consecutive rows of one codebook group (rows_per_cb % 16 == 0) or, when that
// does not hold, a single row.  The codebook is staged in shared memory when it fits.
template <int V, typename IdxT, bool SMEM_CB>
__global__ void __launch_bounds__(256) dequant_bl_kernel(const IdxT* __restrict__ idx,
                                                         const __half* __restrict__ cb,
                                                         __half* __restrict__ w, int N, int K, int C,
                                                         int rows_per_cb, int rows_per_block) {
  using E = typename Entry<V>::T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int J = K / V;
  const int row0 = blockIdx.x * rows_per_block;
  const int group = row0 / rows_per_cb;
  const E* cbg = reinterpret_cast<const E*>(cb) + static_cast<size_t>(group) * C;
  const E* table = cbg;
  if (SMEM_CB) {
    E* s = reinterpret_cast<E*>(smem_raw);
    for (int i = threadIdx.x; i < C; i += blockDim.x) s[i] = cbg[i];
    __syncthreads();
    table = s;
  }
  const int rows = min(rows_per_block, N - row0);
  const long long total = static_cast<long long>(rows) * J;
  const IdxT* ip = idx + static_cast<size_t>(row0) * J;
  E* op = reinterpret_cast<E*>(w + static_cast<size_t>(row0) * K);
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    op[i] = table[min(static_cast<int>(ip[i]), C - 1)];   // an index beyond the codebook reads its last entry
  }
}

// Streaming form, the one normally taken: plain weights (STAGES = 1) and residual weights (STAGES codebook arrays
// and index planes, entries added one after the other in fp16 -- HADD2, round to nearest even, which is the
// residual format's rule).  A block owns a contiguous range of rows, so it rebuilds its
// shared-memory images only when the range crosses into the next codebook group; an image holds every entry
// `reps` times side by side (entry c, replica r at (c * reps + r) * 2V bytes; a lane uses replica lane % reps),
// which makes the lookups conflict-free when reps * 2V = 128 and merely less conflicted when the codebook is too
// large for that.  16 output bytes per thread and step; a warp's stores are one contiguous 512-byte run.
template <int V, typename IdxT> struct IdxWord;                 // the 8/V indices behind 16 output bytes, as one load
template <> struct IdxWord<8, uint8_t> { using T = uint8_t; };
template <> struct IdxWord<8, uint16_t> { using T = uint16_t; };
template <> struct IdxWord<4, uint8_t> { using T = uint16_t; };
template <> struct IdxWord<4, uint16_t> { using T = uint32_t; };
template <> struct IdxWord<2, uint8_t> { using T = uint32_t; };
template <> struct IdxWord<2, uint16_t> { using T = uint2; };

// `cmax` = C - 1: an index beyond the codebook (malformed input) reads the last entry instead of running past
// the image in shared memory.
template <int V, typename IdxT, typename W>
__device__ __forceinline__ uint4 lookup16(const typename Entry<V>::T* tab, W word, int reps, uint32_t cmax) {
  if constexpr (V == 8) {
    return tab[min(static_cast<uint32_t>(word), cmax) * reps];
  } else if constexpr (V == 4) {
    uint32_t c0, c1;
    if constexpr (sizeof(IdxT) == 1) { c0 = word & 0xffu; c1 = word >> 8; }
    else { c0 = word & 0xffffu; c1 = word >> 16; }
    const uint2 e0 = tab[min(c0, cmax) * reps], e1 = tab[min(c1, cmax) * reps];
    return make_uint4(e0.x, e0.y, e1.x, e1.y);
  } else {
    uint32_t c[4];
    if constexpr (sizeof(IdxT) == 1) {
      c[0] = word & 0xffu; c[1] = (word >> 8) & 0xffu; c[2] = (word >> 16) & 0xffu; c[3] = word >> 24;
    } else {
      c[0] = word.x & 0xffffu; c[1] = word.x >> 16; c[2] = word.y & 0xffffu; c[3] = word.y >> 16;
    }
    return make_uint4(tab[min(c[0], cmax) * reps], tab[min(c[1], cmax) * reps], tab[min(c[2], cmax) * reps],
                      tab[min(c[3], cmax) * reps]);
  }
}

// STAGES is a template parameter so that the index loads of a step's four outputs and all their stages are issued
// before the first lookup (with a run-time stage count the loads of one output wait for the lookups of the last).
template <int V, typename IdxT, int STAGES>
__global__ void __launch_bounds__(512) dequant_bl_stream_kernel(const IdxT* __restrict__ idx, const __half* __restrict__ cb,
                                                                __half* __restrict__ w, int N, int K, int C, int rows_per_cb,
                                                                int reps) {
  using E = typename Entry<V>::T;
  using W = typename IdxWord<V, IdxT>::T;
  constexpr int IPT = 8 / V;                   // indices per 16 output bytes
  constexpr int U = 4;                         // outputs per thread and step
  extern __shared__ __align__(16) unsigned char smem_raw[];
  E* img = reinterpret_cast<E*>(smem_raw);
  const int J = K / V;
  const int JO = J / IPT;                      // 16-byte outputs per row
  const int groups = (N + rows_per_cb - 1) / rows_per_cb;
  const size_t plane = static_cast<size_t>(N) * JO;          // index words per stage
  const int img_entries = C * reps;                          // entries of one stage's image
  const int row_lo = static_cast<int>(static_cast<long long>(N) * blockIdx.x / gridDim.x);
  const int row_hi = static_cast<int>(static_cast<long long>(N) * (blockIdx.x + 1) / gridDim.x);
  const E* mine = img + (threadIdx.x & (reps - 1));
  const int nt = blockDim.x;
  const uint32_t cmax = static_cast<uint32_t>(C - 1);
  for (int r0 = row_lo; r0 < row_hi;) {
    const int g = r0 / rows_per_cb;
    const int r1 = min(row_hi, (g + 1) * rows_per_cb);
    __syncthreads();                           // everybody is done with the previous group's images
#pragma unroll
    for (int st = 0; st < STAGES; ++st) {
      const E* src = reinterpret_cast<const E*>(cb) + (static_cast<size_t>(st) * groups + g) * C;
      E* dst = img + static_cast<size_t>(st) * img_entries;
      for (int e = threadIdx.x; e < img_entries; e += nt) dst[e] = __ldg(src + e / reps);
    }
    __syncthreads();
    const long long total = static_cast<long long>(r1 - r0) * JO;
    const W* ip = reinterpret_cast<const W*>(idx) + static_cast<size_t>(r0) * JO;
    uint4* op = reinterpret_cast<uint4*>(w + static_cast<size_t>(r0) * K);
    for (long long i0 = threadIdx.x; i0 < total; i0 += static_cast<long long>(U) * nt) {
      W word[U][STAGES];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * nt;
#pragma unroll
        for (int st = 0; st < STAGES; ++st)
          if (i < total) word[u][st] = __ldg(ip + static_cast<size_t>(st) * plane + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * nt;
        if (i < total) {
          uint4 out = lookup16<V, IdxT, W>(mine, word[u][0], reps, cmax);
#pragma unroll
          for (int st = 1; st < STAGES; ++st) {
            const uint4 e = lookup16<V, IdxT, W>(mine + static_cast<size_t>(st) * img_entries, word[u][st], reps, cmax);
            out.x = hadd2_u32(out.x, e.x); out.y = hadd2_u32(out.y, e.y);
            out.z = hadd2_u32(out.z, e.z); out.w = hadd2_u32(out.w, e.w);
          }
          __stcs(op + i, out);
        }
      }
    }
    r0 = r1;
  }
}

// Launches the streaming kernel when its conditions hold (returns false otherwise, nothing launched):
// v in {2,4,8}, whole 16-byte outputs per row, pointers aligned to what the kernel reads and writes at once,
// and the stages' images fit the shared memory of a block.
static bool launch_stream(const void* idx, const __half* cb, __half* w, int N, int K, int v, int C, int idx_bytes,
                          int rows_per_cb, int stages, cudaStream_t s) {
  if (!(v == 2 || v == 4 || v == 8) || (idx_bytes != 1 && idx_bytes != 2) || stages < 1 || stages > 4) return false;
  const int ipt = 8 / v;
  if ((K / v) % ipt != 0) return false;
  if (reinterpret_cast<uintptr_t>(w) % 16 || reinterpret_cast<uintptr_t>(cb) % (2 * v) ||
      reinterpret_cast<uintptr_t>(idx) % static_cast<uintptr_t>(ipt * idx_bytes))
    return false;
  // a plane of indices must keep that alignment too
  if ((static_cast<size_t>(N) * (K / v) * idx_bytes) % static_cast<size_t>(ipt * idx_bytes) != 0) return false;
  const size_t one = static_cast<size_t>(stages) * C * v * 2;      // unreplicated images
  if (one > 200 * 1024) return false;
  int reps = 64 / v;
  while (reps > 1 && one * reps > 72 * 1024) reps >>= 1;
  const size_t smem = one * reps;
  // two blocks of 512 threads per SM measured best (89 us for 470 MB of weights; three blocks 95, four 102, one 119):
  // enough loads in flight, few enough write streams for the memory's open pages
  int per_sm = static_cast<int>((220 * 1024) / (smem + 1024));
  per_sm = per_sm > 2 ? 2 : (per_sm < 1 ? 1 : per_sm);
  int blocks = 148 * per_sm;
  if (blocks > N) blocks = N;
#define VQG_DQS2(V_, T_, S_)                                                                                  \
  do {                                                                                                        \
    auto k = dequant_bl_stream_kernel<V_, T_, S_>;                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    k<<<blocks, 512, smem, s>>>(static_cast<const T_*>(idx), cb, w, N, K, C, rows_per_cb, reps);              \
  } while (0)
#define VQG_DQS(V_, T_)                                                                                       \
  do {                                                                                                        \
    if (stages == 1) VQG_DQS2(V_, T_, 1); else if (stages == 2) VQG_DQS2(V_, T_, 2);                          \
    else if (stages == 3) VQG_DQS2(V_, T_, 3); else VQG_DQS2(V_, T_, 4);                                      \
  } while (0)
  if (idx_bytes == 1) { if (v == 2) VQG_DQS(2, uint8_t); else if (v == 4) VQG_DQS(4, uint8_t); else VQG_DQS(8, uint8_t); }
  else { if (v == 2) VQG_DQS(2, uint16_t); else if (v == 4) VQG_DQS(4, uint16_t); else VQG_DQS(8, uint16_t); }
#undef VQG_DQS2
#undef VQG_DQS
  return true;
}

// Packed 12-bit indices (two in three bytes): one thread per pair, i.e. three index bytes in and two entries
// (4V bytes, contiguous) out; a warp reads 96 contiguous bytes and writes 64 V.  Same block schedule and images
// as the streaming kernel above (rows are whole numbers of pairs, so a row range is a flat range of pairs).
template <int V>
__global__ void __launch_bounds__(512) dequant_bl_packed12_kernel(const uint8_t* __restrict__ idx, const __half* __restrict__ cb,
                                                                  __half* __restrict__ w, int N, int K, int C, int rows_per_cb,
                                                                  int reps) {
  using E = typename Entry<V>::T;
  constexpr int U = 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  E* img = reinterpret_cast<E*>(smem_raw);
  const int JP = K / V / 2;                    // pairs per row
  const int img_entries = C * reps;
  const int row_lo = static_cast<int>(static_cast<long long>(N) * blockIdx.x / gridDim.x);
  const int row_hi = static_cast<int>(static_cast<long long>(N) * (blockIdx.x + 1) / gridDim.x);
  const E* mine = img + (threadIdx.x & (reps - 1));
  const int nt = blockDim.x;
  for (int r0 = row_lo; r0 < row_hi;) {
    const int g = r0 / rows_per_cb;
    const int r1 = min(row_hi, (g + 1) * rows_per_cb);
    __syncthreads();
    const E* src = reinterpret_cast<const E*>(cb) + static_cast<size_t>(g) * C;
    for (int e = threadIdx.x; e < img_entries; e += nt) img[e] = __ldg(src + e / reps);
    __syncthreads();
    const long long total = static_cast<long long>(r1 - r0) * JP;
    const uint8_t* ip = idx + static_cast<size_t>(r0) * JP * 3;
    E* op = reinterpret_cast<E*>(w + static_cast<size_t>(r0) * K);
    for (long long i0 = threadIdx.x; i0 < total; i0 += static_cast<long long>(U) * nt) {
      uint32_t b[U][3];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * nt;
        if (i < total) {
          b[u][0] = __ldg(ip + 3 * i); b[u][1] = __ldg(ip + 3 * i + 1); b[u][2] = __ldg(ip + 3 * i + 2);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + static_cast<long long>(u) * nt;
        if (i < total) {
          const uint32_t c0 = b[u][0] | ((b[u][1] & 15u) << 8), c1 = (b[u][1] >> 4) | (b[u][2] << 4);
          // 12 bits can name more entries than the codebook has: such an index (malformed input) reads entry 0
          // instead of running past the image
          __stcs(op + 2 * i, mine[(c0 < static_cast<uint32_t>(C) ? c0 : 0u) * reps]);
          __stcs(op + 2 * i + 1, mine[(c1 < static_cast<uint32_t>(C) ? c1 : 0u) * reps]);
        }
      }
    }
    r0 = r1;
  }
}

static int launch_packed12(const uint8_t* idx, const __half* cb, __half* w, int N, int K, int v, int C, int rows_per_cb,
                           cudaStream_t s) {
  if (!(v == 2 || v == 4 || v == 8) || (K / v) % 2 != 0 || C > 4096) return VQG_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(w) % (2 * v) || reinterpret_cast<uintptr_t>(cb) % (2 * v)) return VQG_ERR_BAD_ARG;
  const size_t one = static_cast<size_t>(C) * v * 2;
  int reps = 64 / v;
  while (reps > 1 && one * reps > 72 * 1024) reps >>= 1;
  const size_t smem = one * reps;
  int blocks = 148 * 2;
  if (blocks > N) blocks = N;
#define VQG_DQP(V_)                                                                                           \
  do {                                                                                                        \
    auto k = dequant_bl_packed12_kernel<V_>;                                                                  \
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    k<<<blocks, 512, smem, s>>>(idx, cb, w, N, K, C, rows_per_cb, reps);                                      \
  } while (0)
  if (v == 2) VQG_DQP(2); else if (v == 4) VQG_DQP(4); else VQG_DQP(8);
#undef VQG_DQP
  count_launch();
  return cuda_status(cudaGetLastError());
}

int launch_dequant_bl(const void* idx, const __half* cb, __half* w, int N, int K, int v, int C,
                      int idx_bytes, int rows_per_cb, cudaStream_t s) {
  if (N == 0 || K == 0) return VQG_OK;
  if (idx_bytes == VQG_IDX_PACKED12)
    return launch_packed12(static_cast<const uint8_t*>(idx), cb, w, N, K, v, C, rows_per_cb, s);
  // the kernels read a codebook entry (2v bytes) and write it with one access, and read indices by their own width
  const uintptr_t entry = static_cast<uintptr_t>(2) * static_cast<uintptr_t>(v > 0 ? v : 1);
  if (reinterpret_cast<uintptr_t>(cb) % entry || reinterpret_cast<uintptr_t>(w) % entry ||
      reinterpret_cast<uintptr_t>(idx) % static_cast<uintptr_t>(idx_bytes > 0 ? idx_bytes : 1))
    return VQG_ERR_BAD_ARG;
  const bool single = rows_per_cb >= N;
  int rpb = (single || rows_per_cb % 16 == 0) ? 16 : 1;
  // fewer, larger blocks for large matrices (the codebook is staged once per block)
  while (rpb >= 16 && (single || rows_per_cb % (rpb * 2) == 0) && (N / (rpb * 2)) >= 148 * 16) rpb *= 2;
  const int blocks = (N + rpb - 1) / rpb;
  const size_t cb_bytes = static_cast<size_t>(C) * v * 2;
  if (launch_stream(idx, cb, w, N, K, v, C, idx_bytes, rows_per_cb, 1, s)) {
    count_launch();
    return cuda_status(cudaGetLastError());
  }
  const bool use_smem = cb_bytes <= 96 * 1024;
  const size_t smem = use_smem ? cb_bytes : 0;
#define VQG_DQ(V_, T_)                                                                              \
  do {                                                                                              \
    if (use_smem) {                                                                                 \
      auto k = dequant_bl_kernel<V_, T_, true>;                                                     \
      if (smem > 48 * 1024)                                                                         \
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
      k<<<blocks, 256, smem, s>>>(static_cast<const T_*>(idx), cb, w, N, K, C, rows_per_cb, rpb);   \
    } else {                                                                                        \
      dequant_bl_kernel<V_, T_, false>                                                              \
          <<<blocks, 256, 0, s>>>(static_cast<const T_*>(idx), cb, w, N, K, C, rows_per_cb, rpb);   \
    }                                                                                               \
  } while (0)
  if (idx_bytes == 1) {
    if (v == 2) VQG_DQ(2, uint8_t); else if (v == 4) VQG_DQ(4, uint8_t); else if (v == 8) VQG_DQ(8, uint8_t);
    else return VQG_ERR_UNSUPPORTED;
  } else if (idx_bytes == 2) {
    if (v == 2) VQG_DQ(2, uint16_t); else if (v == 4) VQG_DQ(4, uint16_t); else if (v == 8) VQG_DQ(8, uint16_t);
    else return VQG_ERR_UNSUPPORTED;
  } else {
    return VQG_ERR_UNSUPPORTED;
  }
#undef VQG_DQ
  count_launch();
  return cuda_status(cudaGetLastError());
}

// REF layout, natural orientation: one thread per (k, n); 4-byte gathers, 4-byte stores that
// coalesce along n.
__global__ void __launch_bounds__(256) dequant_ref_kernel(const uint8_t* __restrict__ w,
                                                          const __half* __restrict__ cb,
                                                          __half* __restrict__ out, int Nq, int K) {
  const uint32_t* table = reinterpret_cast<const uint32_t*>(cb);
  uint32_t* o = reinterpret_cast<uint32_t*>(out);
  const long long total = static_cast<long long>(K) * Nq;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(i % Nq);
    o[i] = __ldg(table + (static_cast<size_t>(n >> 2) << 8) + w[i]);
  }
}

// REF layout, transposed output WdecT[2n + r, k]: a 64(k) x 64(n) tile goes through shared
// memory so that both the index reads (along n) and the weight writes (along k) coalesce.
__global__ void __launch_bounds__(256) dequant_ref_t_kernel(const uint8_t* __restrict__ w,
                                                            const __half* __restrict__ cb,
                                                            __half* __restrict__ out, int Nq, int K) {
  __shared__ __half tile[128][66];
  const uint32_t* table = reinterpret_cast<const uint32_t*>(cb);
  const int n0 = blockIdx.x * 64, k0 = blockIdx.y * 64;
  for (int e = threadIdx.x; e < 64 * 64; e += 256) {
    const int kk = e >> 6, nn = e & 63;
    const int k = k0 + kk, n = n0 + nn;
    uint32_t pair = 0;
    if (k < K && n < Nq) pair = __ldg(table + (static_cast<size_t>(n >> 2) << 8) + w[static_cast<size_t>(k) * Nq + n]);
    __half2 h = *reinterpret_cast<__half2*>(&pair);
    tile[2 * nn][kk] = __low2half(h);
    tile[2 * nn + 1][kk] = __high2half(h);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 128 * 64; e += 256) {
    const int r = e >> 6, kk = e & 63;
    const int row = 2 * n0 + r, k = k0 + kk;
    if (row < 2 * Nq && k < K) out[static_cast<size_t>(row) * K + k] = tile[r][kk];
  }
}

// REF layout, streaming form of both orientations.  The reference's format has one 256-entry codebook of 4-byte
// entries per 4 index columns, so a lane that owns ONE codebook (4 consecutive index columns = one 32-bit word of
// an index row) finds its entries in the image [entry c][codebook q] at word c * 32 + q: lane q always reads bank
// q, whatever the indices are, and a warp covers a strip of 32 codebooks = 128 index columns = 256 output columns.
// The image is the strip's 32 KiB of codebooks transposed, nothing is replicated.
//   natural    Wdec [K, 2 Nq]: a lane turns one index word into 16 output bytes; a warp writes 512 contiguous bytes.
//   transposed WdecT [2 Nq, K]: tiles of 64 k.  A lane looks up two k rows (4 columns each), pairs the halves into
//              the 32-bit words (k, k+1) of its 8 output rows and parks them in a [256 rows][32 words] tile; at step s
//              lane l works on k pair (s + l) % 32, which keeps the index reads (bank l), the lookups (bank l) and
//              the tile writes (bank (s + l) % 32) conflict-free.  The tile then leaves in 16-byte stores, 128
//              contiguous bytes per output row.
// A block walks a contiguous range of (strip, 64-k tile) units and rebuilds the image when the strip changes.
constexpr int kRefStripCols = 128;             // index columns per strip
constexpr int kRefTileK = 64;

__device__ __forceinline__ void ref_build_image(const uint32_t* __restrict__ table, uint32_t* image, uint32_t* stage,
                                                int q0, int qs) {
  // codebooks q0 .. q0+qs-1 (1 KiB each, contiguous) -> stage[q][c], then stage -> image[c][q] along diagonals
  const uint4* src = reinterpret_cast<const uint4*>(table + (static_cast<size_t>(q0) << 8));
  uint4* dst = reinterpret_cast<uint4*>(stage);
  for (int e = threadIdx.x; e < qs * 64; e += blockDim.x) dst[e] = __ldg(src + e);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int cb0 = warp * 32; cb0 < 256; cb0 += nwarps * 32) {
    const int c = cb0 + lane;
#pragma unroll 8
    for (int st = 0; st < 32; ++st) {
      const int q = (lane + st) & 31;
      image[c * 32 + q] = q < qs ? stage[q * 256 + c] : 0u;
    }
  }
  __syncthreads();
}

template <bool TRANSPOSED, int NT>
__global__ void __launch_bounds__(NT) dequant_ref_strip_kernel(const uint8_t* __restrict__ w, const __half* __restrict__ cb,
                                                                __half* __restrict__ out, int Nq, int K, int strips,
                                                                int tiles_per_strip) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* image = reinterpret_cast<uint32_t*>(smem_raw);                 // [256][32] words
  uint32_t* otile = image + 256 * 32;                                      // [256 rows][32 words]; staging of the build
  uint32_t* itile = otile + 256 * 32;                                      // [64 k][32 words] (transposed form only)
  const uint32_t* table = reinterpret_cast<const uint32_t*>(cb);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const long long units = static_cast<long long>(strips) * tiles_per_strip;
  const long long u_lo = units * blockIdx.x / gridDim.x, u_hi = units * (blockIdx.x + 1) / gridDim.x;
  int have = -1;
  for (long long u = u_lo; u < u_hi; ++u) {
    const int strip = static_cast<int>(u / tiles_per_strip);
    const int k0 = static_cast<int>(u % tiles_per_strip) * kRefTileK;
    const int k1 = min(K, k0 + kRefTileK);
    const int nq0 = strip * kRefStripCols;
    const int nqs = min(kRefStripCols, Nq - nq0);                          // a multiple of 4
    if (strip != have) {
      __syncthreads();                                                     // the tile is free (previous unit's stores read it)
      ref_build_image(table, image, otile, nq0 >> 2, nqs >> 2);
      have = strip;
    }
    if constexpr (!TRANSPOSED) {
      if (4 * lane < nqs) {
#pragma unroll 4
        for (int k = k0 + warp; k < k1; k += nwarps) {
          const size_t at = static_cast<size_t>(k) * Nq + nq0 + 4 * lane;  // index byte = output word
          const uint32_t four = __ldg(reinterpret_cast<const uint32_t*>(w + at));
          uint4 o;
          o.x = image[(four & 0xffu) * 32 + lane];
          o.y = image[((four >> 8) & 0xffu) * 32 + lane];
          o.z = image[((four >> 16) & 0xffu) * 32 + lane];
          o.w = image[(four >> 24) * 32 + lane];
          __stcs(reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(out) + at), o);
        }
      }
    } else {
      // (1) index tile, coalesced rows of up to 128 bytes
      constexpr int NW = NT / 32;
#pragma unroll
      for (int i = 0; i < kRefTileK / NW; ++i) {
        const int r = warp + NW * i, k = k0 + r;
        uint32_t v = 0;
        if (k < k1 && 4 * lane < nqs) v = __ldg(reinterpret_cast<const uint32_t*>(w + static_cast<size_t>(k) * Nq + nq0 + 4 * lane));
        itile[r * 32 + lane] = v;
      }
      __syncthreads();
      // (2) lookups along diagonals
#pragma unroll
      for (int i = 0; i < 32 / NW; ++i) {
        const int kp = ((32 / NW) * warp + i + lane) & 31;
        const uint32_t a = itile[(2 * kp) * 32 + lane], b = itile[(2 * kp + 1) * 32 + lane];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t ea = image[((a >> (8 * j)) & 0xffu) * 32 + lane];
          const uint32_t eb = image[((b >> (8 * j)) & 0xffu) * 32 + lane];
          otile[(8 * lane + 2 * j) * 32 + kp] = __byte_perm(ea, eb, 0x5410);       // output row 2n  : halves r = 0 of k, k+1
          otile[(8 * lane + 2 * j + 1) * 32 + kp] = __byte_perm(ea, eb, 0x7632);   // output row 2n+1: halves r = 1
        }
      }
      __syncthreads();
      // (3) the tile leaves: 8 lanes write the 128 bytes of one output row
#pragma unroll
      for (int i = 0; i < 2048 / NT; ++i) {
        const int id = threadIdx.x + NT * i;
        const int row = id >> 3, c16 = id & 7;
        const int k = k0 + 8 * c16;
        if (row < 2 * nqs && k < k1) {
          const uint4 v = *reinterpret_cast<const uint4*>(otile + row * 32 + 4 * c16);
          __stcs(reinterpret_cast<uint4*>(out + static_cast<size_t>(2 * nq0 + row) * K + k), v);
        }
      }
      __syncthreads();
    }
  }
}

int launch_dequant_ref(const uint8_t* w, const __half* cb, __half* out, int Nq, int K, bool transposed,
                       cudaStream_t s) {
  if (Nq == 0 || K == 0) return VQG_OK;
  // streaming form: index rows start on 4-byte boundaries (Nq % 4 == 0 holds for the format), 16-byte stores
  if (Nq % 4 == 0 && reinterpret_cast<uintptr_t>(w) % 4 == 0 && reinterpret_cast<uintptr_t>(cb) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(out) % 16 == 0 && (!transposed || K % 8 == 0)) {
    const int strips = (Nq + kRefStripCols - 1) / kRefStripCols;
    const int tiles = (K + kRefTileK - 1) / kRefTileK;
    const long long units = static_cast<long long>(strips) * tiles;
    const int blocks = static_cast<int>(units < 148 * 3 ? units : 148 * 3);   // three blocks of 512 threads per SM
    const size_t smem = transposed ? (32 + 32 + 8) * 1024 : (32 + 32) * 1024;
#define VQG_DQREF(T_, NT_)                                                                              \
  do {                                                                                                  \
    auto k = dequant_ref_strip_kernel<T_, NT_>;                                                         \
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));       \
    k<<<blocks, NT_, smem, s>>>(w, cb, out, Nq, K, strips, tiles);                                      \
  } while (0)
    if (transposed) VQG_DQREF(true, 512); else VQG_DQREF(false, 512);
#undef VQG_DQREF
    count_launch();
    return cuda_status(cudaGetLastError());
  }
  if (transposed) {
    dim3 grid((Nq + 63) / 64, (K + 63) / 64);
    dequant_ref_t_kernel<<<grid, 256, 0, s>>>(w, cb, out, Nq, K);
  } else {
    const long long total = static_cast<long long>(K) * Nq;
    const long long want = (total + 255) / 256;
    const int blocks = static_cast<int>(want < 148LL * 32 ? want : 148LL * 32);
    dequant_ref_kernel<<<blocks, 256, 0, s>>>(w, cb, out, Nq, K);
  }
  count_launch();
  return cuda_status(cudaGetLastError());
}

// fp16 matrix transpose (for `gemm(input, w)` with w given as [K, N]).
__global__ void __launch_bounds__(256) transpose_kernel(const __half* __restrict__ in, __half* __restrict__ out,
                                                        int rows, int cols) {
  __shared__ __half tile[64][66];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  for (int e = threadIdx.x; e < 64 * 64; e += 256) {
    const int rr = e >> 6, cc = e & 63;
    if (r0 + rr < rows && c0 + cc < cols) tile[rr][cc] = in[static_cast<size_t>(r0 + rr) * cols + c0 + cc];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 64 * 64; e += 256) {
    const int cc = e >> 6, rr = e & 63;
    if (r0 + rr < rows && c0 + cc < cols) out[static_cast<size_t>(c0 + cc) * rows + r0 + rr] = tile[rr][cc];
  }
}

int launch_transpose(const __half* in, __half* out, int rows, int cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return VQG_OK;
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  transpose_kernel<<<grid, 256, 0, s>>>(in, out, rows, cols);
  count_launch();
  return cuda_status(cudaGetLastError());
}

// Residual weights: one thread per index position; the stages' entries are added one after the other in fp16
// (HADD2, round to nearest even), which is the format's rule, so the result is bit-exact by construction.
template <int V, typename IdxT>
__global__ void __launch_bounds__(256) dequant_bl_residual_kernel(const IdxT* __restrict__ idx, const __half* __restrict__ cb,
                                                                  __half* __restrict__ w, int N, int K, int C, int rows_per_cb,
                                                                  int stages) {
  const int J = K / V;
  const long long total = static_cast<long long>(N) * J;
  const int groups = (N + rows_per_cb - 1) / rows_per_cb;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(e / J);
    const int g = n / rows_per_cb;
    __half2 acc[V / 2];
#pragma unroll
    for (int r = 0; r < V / 2; ++r)
      acc[r] = reinterpret_cast<const __half2*>(cb + (static_cast<size_t>(g) * C + min(static_cast<int>(idx[e]), C - 1)) * V)[r];
    for (int st = 1; st < stages; ++st) {
      const int cs = min(static_cast<int>(idx[static_cast<size_t>(st) * total + e]), C - 1);
      const __half2* ent = reinterpret_cast<const __half2*>(cb + ((static_cast<size_t>(st) * groups + g) * C + cs) * V);
#pragma unroll
      for (int r = 0; r < V / 2; ++r) acc[r] = __hadd2(acc[r], ent[r]);
    }
#pragma unroll
    for (int r = 0; r < V / 2; ++r) reinterpret_cast<__half2*>(w + e * V)[r] = acc[r];
  }
}

int launch_dequant_bl_residual(const void* idx, const __half* cb, __half* w, int N, int K, int v, int C, int idx_bytes,
                               int rows_per_cb, int stages, cudaStream_t s) {
  if (N == 0 || K == 0) return VQG_OK;
  if (stages < 1 || stages > 8) return VQG_ERR_BAD_ARG;
  if (!(v == 2 || v == 4 || v == 8)) return VQG_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(cb) % 4 || reinterpret_cast<uintptr_t>(w) % 4 ||
      reinterpret_cast<uintptr_t>(idx) % static_cast<uintptr_t>(idx_bytes > 0 ? idx_bytes : 1))
    return VQG_ERR_BAD_ARG;
  if (launch_stream(idx, cb, w, N, K, v, C, idx_bytes, rows_per_cb, stages, s)) {
    count_launch();
    return cuda_status(cudaGetLastError());
  }
  const long long total = static_cast<long long>(N) * (K / v);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
#define VQG_DQR(V_, T_) dequant_bl_residual_kernel<V_, T_><<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const T_*>(idx), cb, w, N, K, C, rows_per_cb, stages)
  if (idx_bytes == 1) { if (v == 2) VQG_DQR(2, uint8_t); else if (v == 4) VQG_DQR(4, uint8_t); else VQG_DQR(8, uint8_t); }
  else if (idx_bytes == 2) { if (v == 2) VQG_DQR(2, uint16_t); else if (v == 4) VQG_DQR(4, uint16_t); else VQG_DQR(8, uint16_t); }
  else return VQG_ERR_UNSUPPORTED;
#undef VQG_DQR
  count_launch();
  return cuda_status(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// Shape-agnostic VQ-GEMM on CUDA cores: 64x64 output tile, 32-wide K steps, 4x4 per thread.
// Accepts any M, N, K (K % v == 0), any C, both layouts.  Not a performance path.
// ---------------------------------------------------------------------------------------------
template <int LAYOUT>
__global__ void __launch_bounds__(256) generic_vq_gemm_kernel(Problem p) {
  __shared__ float xs[32][65];
  __shared__ float ws[32][65];
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  const int J = p.K / p.v;
  const uint8_t* idx8 = static_cast<const uint8_t*>(p.idx);
  const uint16_t* idx16 = static_cast<const uint16_t*>(p.idx);
  for (int k0 = 0; k0 < p.K; k0 += 32) {
    for (int e = threadIdx.x; e < 64 * 32; e += 256) {
      const int r = e >> 5, kk = e & 31;
      const int k = k0 + kk;
      float xv = 0.f, wv = 0.f;
      if (k < p.K) {
        if (m0 + r < p.M) xv = __half2float(p.x[static_cast<size_t>(m0 + r) * p.K + k]);
        const int n = n0 + r;
        if (n < p.N) {
          if (LAYOUT == VQG_LAYOUT_BL) {
            const size_t ii = static_cast<size_t>(n) * J + k / p.v;
            int c;
            if (p.idx_bytes == VQG_IDX_PACKED12) {
              const uint8_t* b = idx8 + 3 * (ii >> 1);
              c = (ii & 1) ? ((b[1] >> 4) | (b[2] << 4)) : (b[0] | ((b[1] & 15) << 8));
            } else {
              c = p.idx_bytes == 1 ? idx8[ii] : idx16[ii];
            }
            c = min(c, p.C - 1);   // this kernel checks the range (the specialised ones trust the caller)
            const int g = n / p.rows_per_cb;
            __half w = p.cb[(static_cast<size_t>(g) * p.C + c) * p.v + (k % p.v)];
            // residual stages: the fp16 running sum of the stages' entries (each addition rounded to fp16)
            const int groups = (p.N + p.rows_per_cb - 1) / p.rows_per_cb;
            for (int st = 1; st < p.n_stages; ++st) {
              const size_t is = static_cast<size_t>(st) * p.N * J + ii;
              const int cs = min(static_cast<int>(p.idx_bytes == 1 ? idx8[is] : idx16[is]), p.C - 1);
              w = __hadd(w, p.cb[((static_cast<size_t>(st) * groups + g) * p.C + cs) * p.v + (k % p.v)]);
            }
            wv = __half2float(w);
          } else {
            const int nq = n >> 1, Nq = p.N >> 1;
            const int c = idx8[static_cast<size_t>(k) * Nq + nq];
            wv = __half2float(p.cb[((static_cast<size_t>(nq >> 2) << 8) + c) * 2 + (n & 1)]);
          }
        }
      }
      xs[kk][r] = xv;
      ws[kk][r] = wv;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = xs[kk][ty * 4 + i]; b[i] = ws[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      const __half h = __float2half_rn(acc[i][j]);
      p.y[static_cast<size_t>(m) * p.ld_y + n] = h;
      for (int q = 0; q < p.n_peers; ++q) p.peer_y[q][static_cast<size_t>(m) * p.ld_y + n] = h;
    }
  }
}

int launch_generic(const Problem& p, int layout, cudaStream_t s) {
  if (p.M == 0 || p.N == 0) return VQG_OK;
  dim3 grid((p.N + 63) / 64, (p.M + 63) / 64);
  if (layout == VQG_LAYOUT_BL) generic_vq_gemm_kernel<VQG_LAYOUT_BL><<<grid, 256, 0, s>>>(p);
  else generic_vq_gemm_kernel<VQG_LAYOUT_REF><<<grid, 256, 0, s>>>(p);
  count_launch();
  return cuda_status(cudaGetLastError());
}

namespace {
// out[m, i] = SiLU(in[m, 2i]) * in[m, 2i+1], fp32 arithmetic on fp16 inputs (the route for shapes the fused
// epilogue does not take)
__global__ void swiglu_kernel(const __half* __restrict__ in, __half* __restrict__ out, int M, int n_out, long long ld_out) {
  const long long total = static_cast<long long>(M) * n_out;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = e / n_out;
    const int i = static_cast<int>(e - m * n_out);
    const float2 gu = __half22float2(*reinterpret_cast<const __half2*>(in + (m * n_out + i) * 2));
    out[m * ld_out + i] = __float2half_rn(gu.x / (1.0f + __expf(-gu.x)) * gu.y);
  }
}
}  // namespace

int launch_swiglu(const __half* in, __half* out, int M, int n_out, long long ld_out, cudaStream_t s) {
  if (M <= 0 || n_out <= 0) return VQG_OK;
  const long long total = static_cast<long long>(M) * n_out;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  swiglu_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(in, out, M, n_out, ld_out);
  count_launch();
  return cuda_status(cudaGetLastError());
}

namespace {
// Row-parallel mode, second step on the owner: y = sum over slots of the ranks' partial blocks.  fp16 in,
// fp32 sum in slot (= rank) order, one rounding; 8 values per thread (16-byte loads).
__global__ void reduce_slots_kernel(const __half* __restrict__ part, __half* __restrict__ y, int slots, int M, int cols,
                                    long long ld_y) {
  const long long vec_per_row = cols / 8;
  const long long total = static_cast<long long>(M) * vec_per_row;
  const long long slot_stride = static_cast<long long>(M) * cols;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = e / vec_per_row;
    const long long c = (e - m * vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < slots; ++s) {
      const uint4 v = *reinterpret_cast<const uint4*>(part + s * slot_stride + m * cols + c);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
    }
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(y + m * ld_y + c) = o;
  }
}

struct OwnerPtrs { __half* p[8]; };
// tmp [M, n_owners*cols] -> block o to owner_part[o] [M, cols]; 16-byte stores (plain, possibly to peer memory)
__global__ void scatter_blocks_kernel(const __half* __restrict__ tmp, OwnerPtrs owners, int n_owners, int M, int cols) {
  const long long vec_per_row = static_cast<long long>(n_owners) * cols / 8;
  const long long total = static_cast<long long>(M) * vec_per_row;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = e / vec_per_row;
    const long long c = (e - m * vec_per_row) * 8;
    const int o = static_cast<int>(c / cols);
    const uint4 v = *reinterpret_cast<const uint4*>(tmp + m * (static_cast<long long>(n_owners) * cols) + c);
    *reinterpret_cast<uint4*>(owners.p[o] + m * cols + (c - static_cast<long long>(o) * cols)) = v;
  }
}
}  // namespace

int launch_reduce_slots(const __half* part, __half* y, int slots, int M, int cols, long long ld_y, cudaStream_t s) {
  if (slots < 1 || M < 0 || cols < 0 || cols % 8 != 0 || ld_y % 8 != 0) return VQG_ERR_BAD_ARG;
  if (M == 0 || cols == 0) return VQG_OK;
  if (reinterpret_cast<uintptr_t>(part) % 16 || reinterpret_cast<uintptr_t>(y) % 16) return VQG_ERR_BAD_ARG;
  const long long total = static_cast<long long>(M) * (cols / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  reduce_slots_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(part, y, slots, M, cols, ld_y);
  count_launch();
  return cuda_status(cudaGetLastError());
}

int launch_scatter_blocks(const __half* tmp, __half* const* owner_part, int n_owners, int M, int cols, cudaStream_t s) {
  if (n_owners < 1 || n_owners > 8 || cols % 8 != 0) return VQG_ERR_BAD_ARG;
  if (M <= 0 || cols <= 0) return VQG_OK;
  OwnerPtrs o{};
  for (int i = 0; i < n_owners; ++i) {
    if (!owner_part[i] || reinterpret_cast<uintptr_t>(owner_part[i]) % 16) return VQG_ERR_BAD_ARG;
    o.p[i] = owner_part[i];
  }
  const long long total = static_cast<long long>(M) * n_owners * (cols / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  scatter_blocks_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(tmp, o, n_owners, M, cols);
  count_launch();
  return cuda_status(cudaGetLastError());
}

}  // namespace vqg
