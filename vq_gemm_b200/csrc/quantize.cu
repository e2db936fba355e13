// The step before the product: turning a dense fp16 weight matrix W[N, K] into (indices, codebooks) of the
// generalised format, on the GPU.  The reference has no quantiser (bench.py:83-85 draws random indices).
//
//   assign   idx[n, j] = argmin_c d(W[n, jv : jv+v], cb[g(n)][c]),  lowest c among equal distances
//            d(a, b) = sum_i (float(a_i) - float(b_i))^2, i ascending, every subtract, multiply and add
//            rounded to fp32 on its own (no fused multiply-add) -- a rule a CPU can restate bit for bit
//   update   cb[g][c] = mean of the sub-vectors assigned to (g, c); entries nobody chose keep their value.
//            Sums are EXACT and order-independent: every finite fp16 is an integer multiple of 2^-24, so the
//            kernel adds 64-bit integers (value * 2^24); mean = float(double(sum) * 2^-24 / count) -> fp16.
//   pack12 / unpack12   two 12-bit indices <-> three bytes (little end first), for codebooks of 4096 entries
//            whose indices otherwise sit in uint16 with four unused bits each.
//
// All three are CUDA-core kernels: the distance search is bound by the fp32 pipe (3v lane operations per
// (sub-vector, entry) pair), the update by shared-memory atomics (native 32-bit ones where the accumulators fit,
// see accumulate_split_kernel), the packers by HBM.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"

namespace vqg {
namespace {

constexpr int kAssignThreads = 256;
constexpr int kSubPerThread = 2;       // independent searches per thread (instruction-level parallelism)

template <int V>
__device__ __forceinline__ void load_sub(const __half* p, float (&out)[V]) {
  if constexpr (V == 8) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
  } else if constexpr (V == 4) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 2; ++i) { const float2 f = __half22float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
  } else {
    const uint32_t r = __ldg(reinterpret_cast<const uint32_t*>(p));
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r));
    out[0] = f.x; out[1] = f.y;
  }
}

// grid (chunks, groups); the CTA searches the sub-vectors of its group, kAssignThreads * kSubPerThread at a time
template <int V, typename IdxT>
__global__ void __launch_bounds__(kAssignThreads)
assign_kernel(const __half* __restrict__ w, const __half* __restrict__ cb, IdxT* __restrict__ idx, int N, int K, int C,
              int rows_per_cb) {
  extern __shared__ float s_cb[];   // [C][V] fp32
  const int g = blockIdx.y;
  const __half* cbg = cb + static_cast<size_t>(g) * C * V;
  for (int i = threadIdx.x; i < C * V; i += kAssignThreads) s_cb[i] = __half2float(cbg[i]);
  __syncthreads();
  const int J = K / V;
  const int row0 = g * rows_per_cb;
  const int rows = min(rows_per_cb, N - row0);
  const long long total = static_cast<long long>(rows) * J;                 // sub-vectors of the group
  const long long base = static_cast<long long>(row0) * J;
  const long long stride = static_cast<long long>(gridDim.x) * kAssignThreads * kSubPerThread;
  for (long long s0 = static_cast<long long>(blockIdx.x) * kAssignThreads * kSubPerThread; s0 < total; s0 += stride) {
    float x[kSubPerThread][V];
    long long pos[kSubPerThread];
#pragma unroll
    for (int u = 0; u < kSubPerThread; ++u) {
      pos[u] = s0 + u * kAssignThreads + threadIdx.x;
      if (pos[u] < total) load_sub<V>(w + (base + pos[u]) * V, x[u]);
      else {
#pragma unroll
        for (int i = 0; i < V; ++i) x[u][i] = 0.f;
      }
    }
    float best[kSubPerThread];
    int arg[kSubPerThread];
#pragma unroll
    for (int u = 0; u < kSubPerThread; ++u) { best[u] = __int_as_float(0x7f800000); arg[u] = 0; }
#pragma unroll 2
    for (int c = 0; c < C; ++c) {
      float e[V];
      if constexpr (V == 8) {
        const float4 a = *reinterpret_cast<const float4*>(s_cb + c * 8), b = *reinterpret_cast<const float4*>(s_cb + c * 8 + 4);
        e[0] = a.x; e[1] = a.y; e[2] = a.z; e[3] = a.w; e[4] = b.x; e[5] = b.y; e[6] = b.z; e[7] = b.w;
      } else if constexpr (V == 4) {
        const float4 a = *reinterpret_cast<const float4*>(s_cb + c * 4);
        e[0] = a.x; e[1] = a.y; e[2] = a.z; e[3] = a.w;
      } else {
        const float2 a = *reinterpret_cast<const float2*>(s_cb + c * 2);
        e[0] = a.x; e[1] = a.y;
      }
#pragma unroll
      for (int u = 0; u < kSubPerThread; ++u) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float t = __fsub_rn(x[u][i], e[i]);
          d = __fadd_rn(d, __fmul_rn(t, t));
        }
        if (d < best[u]) { best[u] = d; arg[u] = c; }   // strict: the lowest index wins a tie
      }
    }
#pragma unroll
    for (int u = 0; u < kSubPerThread; ++u)
      if (pos[u] < total) idx[base + pos[u]] = static_cast<IdxT>(arg[u]);
  }
}

// The same search with Blackwell's packed fp32 arithmetic (sub / mul / add .f32x2: two IEEE operations per
// instruction, each rounded exactly like its scalar form, so the results are the same bits): a thread searches
// eight sub-vectors as four packed pairs; the codebook sits in shared memory with every value doubled -- (e, e) -- so
// that an entry's operands arrive as ready 64-bit pairs.  Needs C * V * 8 bytes of shared memory.
__device__ __forceinline__ unsigned long long f2_sub(unsigned long long a, unsigned long long b) {
  unsigned long long r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ unsigned long long f2_mul(unsigned long long a, unsigned long long b) {
  unsigned long long r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
  unsigned long long r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ unsigned long long f2_pack(float lo, float hi) {
  return static_cast<unsigned long long>(__float_as_uint(lo)) | (static_cast<unsigned long long>(__float_as_uint(hi)) << 32);
}

constexpr int kPairsPerThread = 4;     // packed pairs (eight sub-vectors) per thread
template <int V, typename IdxT>
__global__ void __launch_bounds__(kAssignThreads)
assign_packed_kernel(const __half* __restrict__ w, const __half* __restrict__ cb, IdxT* __restrict__ idx, int N, int K, int C,
                     int rows_per_cb) {
  extern __shared__ __align__(16) unsigned long long s_cb2[];   // [C][V] pairs (e, e)
  const int g = blockIdx.y;
  const __half* cbg = cb + static_cast<size_t>(g) * C * V;
  for (int i = threadIdx.x; i < C * V; i += kAssignThreads) {
    const float e = __half2float(cbg[i]);
    s_cb2[i] = f2_pack(e, e);
  }
  __syncthreads();
  const int J = K / V;
  const int row0 = g * rows_per_cb;
  const int rows = min(rows_per_cb, N - row0);
  const long long total = static_cast<long long>(rows) * J;
  const long long base = static_cast<long long>(row0) * J;
  constexpr int SUBS = 2 * kPairsPerThread;
  const long long stride = static_cast<long long>(gridDim.x) * kAssignThreads * SUBS;
  for (long long s0 = static_cast<long long>(blockIdx.x) * kAssignThreads * SUBS; s0 < total; s0 += stride) {
    long long pos[SUBS];
    unsigned long long x2[kPairsPerThread][V];
#pragma unroll
    for (int p = 0; p < kPairsPerThread; ++p) {
      float xa[V], xb[V];
      pos[2 * p] = s0 + (2 * p) * kAssignThreads + threadIdx.x;
      pos[2 * p + 1] = s0 + (2 * p + 1) * kAssignThreads + threadIdx.x;
#pragma unroll
      for (int i = 0; i < V; ++i) { xa[i] = 0.f; xb[i] = 0.f; }
      if (pos[2 * p] < total) load_sub<V>(w + (base + pos[2 * p]) * V, xa);
      if (pos[2 * p + 1] < total) load_sub<V>(w + (base + pos[2 * p + 1]) * V, xb);
#pragma unroll
      for (int i = 0; i < V; ++i) x2[p][i] = f2_pack(xa[i], xb[i]);
    }
    float best[SUBS];
    int arg[SUBS];
#pragma unroll
    for (int u = 0; u < SUBS; ++u) { best[u] = __int_as_float(0x7f800000); arg[u] = 0; }
#pragma unroll 2
    for (int c = 0; c < C; ++c) {
      unsigned long long e2[V];
#pragma unroll
      for (int i = 0; i < V; i += 2) {
        const ulonglong2 q = *reinterpret_cast<const ulonglong2*>(s_cb2 + c * V + i);
        e2[i] = q.x; e2[i + 1] = q.y;
      }
#pragma unroll
      for (int p = 0; p < kPairsPerThread; ++p) {
        unsigned long long d2 = 0ull;              // (+0, +0)
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const unsigned long long t = f2_sub(x2[p][i], e2[i]);
          d2 = f2_add(d2, f2_mul(t, t));
        }
        const float da = __uint_as_float(static_cast<unsigned int>(d2)), db = __uint_as_float(static_cast<unsigned int>(d2 >> 32));
        if (da < best[2 * p]) { best[2 * p] = da; arg[2 * p] = c; }           // strict: the lowest index wins a tie
        if (db < best[2 * p + 1]) { best[2 * p + 1] = db; arg[2 * p + 1] = c; }
      }
    }
#pragma unroll
    for (int u = 0; u < SUBS; ++u)
      if (pos[u] < total) idx[base + pos[u]] = static_cast<IdxT>(arg[u]);
  }
}

constexpr int kAccThreads = 256;

// value * 2^24 as a two's-complement 64-bit integer: exact for every finite fp16 (|value| <= 65504, smallest
// step 2^-24; the fp32 product keeps the 11 significant bits)
__device__ __forceinline__ unsigned long long to_fixed(float fp16_value) {
  return static_cast<unsigned long long>(static_cast<long long>(fp16_value * 16777216.0f));
}

// grid (chunks, groups).  SMEM: per-CTA accumulators in shared memory, flushed once; otherwise global atomics.
template <int V, typename IdxT, bool SMEM>
__global__ void __launch_bounds__(kAccThreads)
accumulate_kernel(const __half* __restrict__ w, const IdxT* __restrict__ idx, unsigned long long* __restrict__ sums,
                  unsigned int* __restrict__ counts, int N, int K, int C, int rows_per_cb) {
  extern __shared__ unsigned long long s_acc[];   // [C][V] sums, then [C] counts (32-bit)
  unsigned int* s_cnt = reinterpret_cast<unsigned int*>(s_acc + static_cast<size_t>(C) * V);
  const int g = blockIdx.y;
  if (SMEM) {
    for (int i = threadIdx.x; i < C * V; i += kAccThreads) s_acc[i] = 0ull;
    for (int i = threadIdx.x; i < C; i += kAccThreads) s_cnt[i] = 0u;
    __syncthreads();
  }
  const int J = K / V;
  const int row0 = g * rows_per_cb;
  const int rows = min(rows_per_cb, N - row0);
  const long long total = static_cast<long long>(rows) * J;
  const long long base = static_cast<long long>(row0) * J;
  unsigned long long* gs = sums + static_cast<size_t>(g) * C * V;
  unsigned int* gc = counts + static_cast<size_t>(g) * C;
  for (long long s = static_cast<long long>(blockIdx.x) * kAccThreads + threadIdx.x; s < total;
       s += static_cast<long long>(gridDim.x) * kAccThreads) {
    const int c = static_cast<int>(idx[base + s]);
    if (c >= C) continue;            // foreign index: ignored (the product's kernels would read past the codebook)
    float x[V];
    load_sub<V>(w + (base + s) * V, x);
    if (SMEM) {
#pragma unroll
      for (int i = 0; i < V; ++i) atomicAdd(&s_acc[c * V + i], to_fixed(x[i]));
      atomicAdd(&s_cnt[c], 1u);
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) atomicAdd(&gs[c * V + i], to_fixed(x[i]));
      atomicAdd(&gc[c], 1u);
    }
  }
  if (SMEM) {
    __syncthreads();
    for (int i = threadIdx.x; i < C * V; i += kAccThreads)
      if (s_acc[i] != 0ull) atomicAdd(&gs[i], s_acc[i]);
    for (int i = threadIdx.x; i < C; i += kAccThreads)
      if (s_cnt[i] != 0u) atomicAdd(&gc[i], s_cnt[i]);
  }
}

// The same sums with native 32-bit shared-memory atomics (64-bit ones are compare-and-swap loops): a value's
// fixed-point form f (|f| < 2^40) is split into a signed low part lo in [-2^20, 2^20) and hi = (f - lo) / 2^21,
// each added into its own 32-bit counter.  hi is zero for |value| < 1/16, i.e. for nearly every weight of a real
// layer, and then costs nothing.  A CTA works in rounds of kRound = 2048 sub-vectors -- after which a counter holds
// at most 2048 * 2^20 = 2^31 in magnitude, exactly what fits -- and folds the counters into 64-bit totals (one owner
// thread per address, no atomics) between rounds.  The counters are laid out [dimension][entry], so that a warp's
// atomics on one dimension spread over all banks.  Exact and order-independent like the rule asks.
constexpr int kRound = 2048;
template <int V, typename IdxT>
__global__ void __launch_bounds__(kAccThreads)
accumulate_split_kernel(const __half* __restrict__ w, const IdxT* __restrict__ idx, unsigned long long* __restrict__ sums,
                        unsigned int* __restrict__ counts, int N, int K, int C, int rows_per_cb) {
  extern __shared__ unsigned long long s_tot[];   // [C][V] totals, then lo [C][V], hi [C][V], counts [C] (32-bit each)
  const int CV = C * V;
  int* s_lo = reinterpret_cast<int*>(s_tot + CV);
  int* s_hi = s_lo + CV;
  unsigned int* s_cnt = reinterpret_cast<unsigned int*>(s_hi + CV);
  const int g = blockIdx.y;
  for (int i = threadIdx.x; i < CV; i += kAccThreads) { s_tot[i] = 0ull; s_lo[i] = 0; s_hi[i] = 0; }
  for (int i = threadIdx.x; i < C; i += kAccThreads) s_cnt[i] = 0u;
  __syncthreads();
  const int J = K / V;
  const int row0 = g * rows_per_cb;
  const int rows = min(rows_per_cb, N - row0);
  const long long total = static_cast<long long>(rows) * J;
  const long long base = static_cast<long long>(row0) * J;
  constexpr int U = kRound / kAccThreads;          // sub-vectors per thread and round
  for (long long s0 = static_cast<long long>(blockIdx.x) * kRound; s0 < total; s0 += static_cast<long long>(gridDim.x) * kRound) {
    int c[U];
    float x[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long sv = s0 + u * kAccThreads + threadIdx.x;
      c[u] = C;                                    // "nothing": beyond the range, or a foreign index
      if (sv < total) {
        c[u] = static_cast<int>(idx[base + sv]);
        load_sub<V>(w + (base + sv) * V, x[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (c[u] < C) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const long long f = static_cast<long long>(x[u][i] * 16777216.0f);
          const int lo = static_cast<int>((f + (1ll << 20)) & ((1ll << 21) - 1)) - (1 << 20);
          const int hi = static_cast<int>((f - lo) >> 21);
          atomicAdd(&s_lo[i * C + c[u]], lo);
          if (hi != 0) atomicAdd(&s_hi[i * C + c[u]], hi);
        }
        atomicAdd(&s_cnt[c[u]], 1u);
      }
    }
    __syncthreads();
    for (int a = threadIdx.x; a < CV; a += kAccThreads) {      // a = i * C + c in the counters, c * V + i in the totals
      const long long add = static_cast<long long>(s_hi[a]) * (1ll << 21) + static_cast<long long>(s_lo[a]);
      s_tot[(a % C) * V + a / C] += static_cast<unsigned long long>(add);
      s_lo[a] = 0;
      s_hi[a] = 0;
    }
    __syncthreads();
  }
  unsigned long long* gs = sums + static_cast<size_t>(g) * CV;
  unsigned int* gc = counts + static_cast<size_t>(g) * C;
  for (int i = threadIdx.x; i < CV; i += kAccThreads)
    if (s_tot[i] != 0ull) atomicAdd(&gs[i], s_tot[i]);
  for (int i = threadIdx.x; i < C; i += kAccThreads)
    if (s_cnt[i] != 0u) atomicAdd(&gc[i], s_cnt[i]);
}

__global__ void finalize_kernel(__half* __restrict__ cb, const unsigned long long* __restrict__ sums,
                                const unsigned int* __restrict__ counts, long long entries, int V) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;   // (g, c)
  if (e >= entries) return;
  const unsigned int n = counts[e];
  if (n == 0u) return;               // nobody chose the entry: it keeps its value
  for (int i = 0; i < V; ++i) {
    const long long sum = static_cast<long long>(sums[e * V + i]);
    const double mean = static_cast<double>(sum) * (1.0 / 16777216.0) / static_cast<double>(n);
    cb[e * V + i] = __float2half_rn(static_cast<float>(mean));
  }
}

// two 12-bit values a, b -> bytes [a & 255, (a >> 8) | ((b & 15) << 4), b >> 4]
__global__ void pack12_kernel(const uint16_t* __restrict__ in, unsigned char* __restrict__ out, long long pairs) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t two = __ldg(reinterpret_cast<const uint32_t*>(in) + i);
    const uint32_t a = two & 0xfffu, b = (two >> 16) & 0xfffu;
    const uint32_t packed = a | (b << 12);
    unsigned char* o = out + 3 * i;
    o[0] = static_cast<unsigned char>(packed);
    o[1] = static_cast<unsigned char>(packed >> 8);
    o[2] = static_cast<unsigned char>(packed >> 16);
  }
}

__global__ void unpack12_kernel(const unsigned char* __restrict__ in, uint16_t* __restrict__ out, long long pairs) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned char* p = in + 3 * i;
    const uint32_t packed = static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) | (static_cast<uint32_t>(p[2]) << 16);
    reinterpret_cast<uint32_t*>(out)[i] = (packed & 0xfffu) | ((packed >> 12) << 16);
  }
}

// Wide forms: a thread moves 16 indices -- 32 bytes of uint16 (two 16-byte accesses) against 24 packed bytes
// (three 8-byte accesses); both sides 16- / 8-byte aligned, the tail (fewer than 16 indices) goes to the kernels above.
__global__ void __launch_bounds__(256) pack12_wide_kernel(const uint4* __restrict__ in, uint2* __restrict__ out, long long groups) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < groups;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 a = __ldcs(in + 2 * i), b = __ldcs(in + 2 * i + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t p[8];                       // 24 bits each: the pair (lo12, hi12) of one input word
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = (w[j] & 0xfffu) | (((w[j] >> 16) & 0xfffu) << 12);
    // eight 24-bit groups -> six 32-bit words
    uint32_t o[6];
    o[0] = p[0] | (p[1] << 24);
    o[1] = (p[1] >> 8) | (p[2] << 16);
    o[2] = (p[2] >> 16) | (p[3] << 8);
    o[3] = p[4] | (p[5] << 24);
    o[4] = (p[5] >> 8) | (p[6] << 16);
    o[5] = (p[6] >> 16) | (p[7] << 8);
    __stcs(out + 3 * i, make_uint2(o[0], o[1]));
    __stcs(out + 3 * i + 1, make_uint2(o[2], o[3]));
    __stcs(out + 3 * i + 2, make_uint2(o[4], o[5]));
  }
}

__global__ void __launch_bounds__(256) unpack12_wide_kernel(const uint2* __restrict__ in, uint4* __restrict__ out, long long groups) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < groups;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint2 a = __ldcs(in + 3 * i), b = __ldcs(in + 3 * i + 1), c = __ldcs(in + 3 * i + 2);
    const uint32_t o[6] = {a.x, a.y, b.x, b.y, c.x, c.y};
    uint32_t p[8];
    p[0] = o[0] & 0xffffffu;
    p[1] = ((o[0] >> 24) | (o[1] << 8)) & 0xffffffu;
    p[2] = ((o[1] >> 16) | (o[2] << 16)) & 0xffffffu;
    p[3] = o[2] >> 8;
    p[4] = o[3] & 0xffffffu;
    p[5] = ((o[3] >> 24) | (o[4] << 8)) & 0xffffffu;
    p[6] = ((o[4] >> 16) | (o[5] << 16)) & 0xffffffu;
    p[7] = o[5] >> 8;
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = (p[j] & 0xfffu) | ((p[j] >> 12) << 16);
    __stcs(out + 2 * i, make_uint4(w[0], w[1], w[2], w[3]));
    __stcs(out + 2 * i + 1, make_uint4(w[4], w[5], w[6], w[7]));
  }
}

int groups_of(int N, int rows_per_cb) { return rows_per_cb >= N ? 1 : (N + rows_per_cb - 1) / rows_per_cb; }

int sm_count_q() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

bool quantize_args_ok(const void* w, int N, int K, int v, int C, int idx_bytes) {
  if (!(v == 2 || v == 4 || v == 8) || K % v != 0) return false;
  if (C < 1 || C > 65536 || (idx_bytes != 1 && idx_bytes != 2) || (idx_bytes == 1 && C > 256)) return false;
  if (reinterpret_cast<uintptr_t>(w) % 16 != 0) return false;   // sub-vectors are read with one aligned load each
  return N > 0 && K > 0;
}

}  // namespace

size_t quantize_workspace_bytes(int N, int v, int C, int rows_per_cb) {
  const int rpc = (rows_per_cb <= 0 || rows_per_cb > N) ? N : rows_per_cb;
  const size_t entries = static_cast<size_t>(groups_of(N, rpc)) * C;
  return entries * v * sizeof(unsigned long long) + entries * sizeof(unsigned int);
}

int launch_quantize_assign(const __half* w, const __half* cb, void* idx, int N, int K, int v, int C, int idx_bytes,
                           int rows_per_cb, cudaStream_t s) {
  if (!quantize_args_ok(w, N, K, v, C, idx_bytes)) return VQG_ERR_UNSUPPORTED;
  const int rpc = (rows_per_cb <= 0 || rows_per_cb > N) ? N : rows_per_cb;
  const int G = groups_of(N, rpc);
  const bool packed = static_cast<size_t>(C) * v * 8 <= 200 * 1024;      // the doubled codebook fits: packed fp32 arithmetic
  const size_t smem = static_cast<size_t>(C) * v * (packed ? 8 : sizeof(float));
  if (smem > 200 * 1024) return VQG_ERR_UNSUPPORTED;
  const long long per_group = static_cast<long long>(rpc) * (K / v);
  const long long per_cta = static_cast<long long>(kAssignThreads) * (packed ? 2 * kPairsPerThread : kSubPerThread);
  long long chunks = (per_group + per_cta - 1) / per_cta;
  const long long want = (4LL * sm_count_q() + G - 1) / G;     // about four CTAs per SM in total
  if (chunks > want) chunks = want;
  if (chunks < 1) chunks = 1;
  const dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(G));
#define VQG_ASSIGN(VV, TT)                                                                                       \
  do {                                                                                                           \
    auto kern = packed ? assign_packed_kernel<VV, TT> : assign_kernel<VV, TT>;                                   \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) \
      return VQG_ERR_LAUNCH;                                                                                     \
    kern<<<grid, kAssignThreads, smem, s>>>(w, cb, static_cast<TT*>(idx), N, K, C, rpc);                         \
  } while (0)
  if (idx_bytes == 1) {
    if (v == 8) VQG_ASSIGN(8, unsigned char); else if (v == 4) VQG_ASSIGN(4, unsigned char); else VQG_ASSIGN(2, unsigned char);
  } else {
    if (v == 8) VQG_ASSIGN(8, uint16_t); else if (v == 4) VQG_ASSIGN(4, uint16_t); else VQG_ASSIGN(2, uint16_t);
  }
#undef VQG_ASSIGN
  count_launch();
  note_weights_written(s);
  return cuda_status(cudaGetLastError());
}

int launch_quantize_update(const __half* w, const void* idx, __half* cb, void* ws, size_t ws_bytes, int N, int K, int v,
                           int C, int idx_bytes, int rows_per_cb, cudaStream_t s) {
  if (!quantize_args_ok(w, N, K, v, C, idx_bytes)) return VQG_ERR_UNSUPPORTED;
  const size_t need = quantize_workspace_bytes(N, v, C, rows_per_cb);
  if (!ws || ws_bytes < need || reinterpret_cast<uintptr_t>(ws) % 16 != 0) return VQG_ERR_WORKSPACE;
  const int rpc = (rows_per_cb <= 0 || rows_per_cb > N) ? N : rows_per_cb;
  const int G = groups_of(N, rpc);
  const size_t entries = static_cast<size_t>(G) * C;
  unsigned long long* sums = static_cast<unsigned long long*>(ws);
  unsigned int* counts = reinterpret_cast<unsigned int*>(sums + entries * v);
  if (cudaMemsetAsync(ws, 0, need, s) != cudaSuccess) return VQG_ERR_LAUNCH;
  const size_t smem = static_cast<size_t>(C) * v * sizeof(unsigned long long) + static_cast<size_t>(C) * sizeof(unsigned int);
  const bool in_smem = smem <= 160 * 1024;
  const size_t smem_split = static_cast<size_t>(C) * v * 16 + static_cast<size_t>(C) * sizeof(unsigned int);
  const bool split = smem_split <= 200 * 1024;
  const long long per_group = static_cast<long long>(rpc) * (K / v);
  long long chunks = (per_group + 16LL * kAccThreads - 1) / (16LL * kAccThreads);
  const long long want = (2LL * sm_count_q() + G - 1) / G;
  if (chunks > want) chunks = want;
  if (chunks < 1) chunks = 1;
  const dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(G));
#define VQG_ACC(VV, TT)                                                                                              \
  do {                                                                                                               \
    if (split) {                                                                                                     \
      if (cudaFuncSetAttribute(accumulate_split_kernel<VV, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                               static_cast<int>(smem_split)) != cudaSuccess)                                         \
        return VQG_ERR_LAUNCH;                                                                                       \
      accumulate_split_kernel<VV, TT><<<grid, kAccThreads, smem_split, s>>>(w, static_cast<const TT*>(idx), sums, counts, \
                                                                            N, K, C, rpc);                            \
    } else if (in_smem) {                                                                                            \
      if (cudaFuncSetAttribute(accumulate_kernel<VV, TT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                               static_cast<int>(smem)) != cudaSuccess)                                               \
        return VQG_ERR_LAUNCH;                                                                                       \
      accumulate_kernel<VV, TT, true><<<grid, kAccThreads, smem, s>>>(w, static_cast<const TT*>(idx), sums, counts, N, K, \
                                                                      C, rpc);                                        \
    } else {                                                                                                         \
      accumulate_kernel<VV, TT, false><<<grid, kAccThreads, 0, s>>>(w, static_cast<const TT*>(idx), sums, counts, N, K, C, \
                                                                    rpc);                                             \
    }                                                                                                                \
  } while (0)
  if (idx_bytes == 1) {
    if (v == 8) VQG_ACC(8, unsigned char); else if (v == 4) VQG_ACC(4, unsigned char); else VQG_ACC(2, unsigned char);
  } else {
    if (v == 8) VQG_ACC(8, uint16_t); else if (v == 4) VQG_ACC(4, uint16_t); else VQG_ACC(2, uint16_t);
  }
#undef VQG_ACC
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return VQG_ERR_LAUNCH;
  const long long n_entries = static_cast<long long>(entries);
  finalize_kernel<<<static_cast<unsigned>((n_entries + 255) / 256), 256, 0, s>>>(cb, sums, counts, n_entries, v);
  count_launch();
  note_weights_written(s);
  return cuda_status(cudaGetLastError());
}

int launch_pack12(const void* in, void* out, long long values, bool pack, cudaStream_t s) {
  if (values < 0 || values % 2 != 0) return VQG_ERR_BAD_ARG;
  if (values == 0) return VQG_OK;
  const void* two_byte_side = pack ? in : out;
  if (reinterpret_cast<uintptr_t>(two_byte_side) % 4 != 0) return VQG_ERR_BAD_ARG;
  const long long cap = 32LL * sm_count_q();
  const unsigned char* packed_side = static_cast<const unsigned char*>(pack ? out : in);
  long long done = 0;                                   // indices handled by the wide kernel
  if (values >= 16 && reinterpret_cast<uintptr_t>(two_byte_side) % 16 == 0 && reinterpret_cast<uintptr_t>(packed_side) % 8 == 0) {
    const long long groups = values / 16;
    long long blocks = (groups + 255) / 256;
    if (blocks > cap) blocks = cap;
    if (pack)
      pack12_wide_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const uint4*>(in), static_cast<uint2*>(out), groups);
    else
      unpack12_wide_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const uint2*>(in), static_cast<uint4*>(out), groups);
    count_launch();
    done = groups * 16;
  }
  const long long pairs = (values - done) / 2;
  if (pairs > 0) {
    long long blocks = (pairs + 255) / 256;
    if (blocks > cap) blocks = cap;
    const uint16_t* u16 = static_cast<const uint16_t*>(two_byte_side) + done;
    const unsigned char* pk = packed_side + done / 2 * 3;
    if (pack)
      pack12_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(u16, const_cast<unsigned char*>(pk), pairs);
    else
      unpack12_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(pk, const_cast<uint16_t*>(u16), pairs);
    count_launch();
  }
  note_weights_written(s);
  return cuda_status(cudaGetLastError());
}

}  // namespace vqg
