// Memory-bound VQ-GEMM for M <= 16 (decode / small batch), sm_100a.
//
// The problem is a GEMV-like stream over the index matrix: every index is read once from HBM
// and costs one shared-memory codebook lookup.  The kernel is persistent (one 512-thread CTA per
// SM) and works on items of 16 output rows x up to 4096 K values:
//
//   * indices are streamed with 64-/128-bit loads straight into registers, two items ahead
//     of use (register ring), so ~32 KiB per SM are in flight;
//   * the codebook of the item's group sits in shared memory as a REPLICATED image: entry c,
//     replica r at byte  c*(R*2v) + r*2v , lane uses replica lane % R.  With R = 64/v
//     (C <= 256) a warp-wide lookup touches every bank exactly once per wavefront;
//   * a looked-up entry IS an mma.sync A fragment: with the K values of an m16n8k16 step
//     permuted so that thread (g, t) owns 4 consecutive K values of rows g and g+8, the 8
//     (v=4) or 16 (v=8) bytes of an entry drop into the fragment registers without any
//     conversion or shuffle.  X is the B operand (batch padded to 8 or 16 columns) and lives
//     in registers for the whole kernel; accumulation is fp32 in the tensor core;
//   * each warp owns a 256-wide K slice; the 16 partial tiles of a CTA are summed in a fixed
//     order through shared memory (deterministic), and K > 4096 adds a split-K step through a
//     caller-provided workspace in which the last-arriving CTA of a row block sums the chunks
//     in chunk order (also deterministic).
//
// There is no reference counterpart: the reference requires M % 128 == 0
// (strategy_1/src.cu:221).
#include <mutex>

#include "common.cuh"

namespace vqg {

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = 16;
constexpr int kSliceK = 256;     // K values per warp slice
constexpr int kRedStride = 20;   // floats per batch column in the reduction buffer (16 rows + pad)
constexpr int kPrefetch = 3;     // index register ring depth

struct DecodeParams {
  const __half* x;
  const void* idx;
  const __half* cb;
  __half* y;
  float* ws_partial;   // [nchunks][M][N] fp32 (split-K only)
  int* ws_counter;     // [items per chunk]
  int* status;
  int M, N, K, C;
  int rows_per_cb;
  long long ld_y;
  int nslices;         // K / 256
  int nchunks;         // ceil(nslices / 16)
  int rl;              // 16-row blocks processed side by side by one CTA
  int nrbg;            // N / (16 * rl)
  int rep_log2;        // log2 of codebook replicas
  int n_peers;
  __half* peer_y[8];
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int WORDS>
struct IdxRegs { uint32_t w[WORDS]; };

template <int WORDS>
__device__ __forceinline__ void load_idx(IdxRegs<WORDS>& r, const void* p) {
  if constexpr (WORDS == 2) {
    uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    r.w[0] = t.x; r.w[1] = t.y;
  } else {
#pragma unroll
    for (int i = 0; i < WORDS / 4; ++i) {
      uint4 t = __ldcs(reinterpret_cast<const uint4*>(p) + i);
      r.w[4 * i] = t.x; r.w[4 * i + 1] = t.y; r.w[4 * i + 2] = t.z; r.w[4 * i + 3] = t.w;
    }
  }
}

// V: sub-vector length (4 or 8); IB: index bytes (1 or 2); MB: batch tiles of 8 (1 or 2).
template <int V, int IB, int MB>
__global__ void __launch_bounds__(kThreads, 1) vq_decode_kernel(const DecodeParams p) {
  constexpr int IPT = 64 / V;              // indices per thread per row per item
  constexpr int WORDS = IPT * IB / 4;      // 32-bit words of indices per row
  constexpr int ENTRY_LOG2 = (V == 4) ? 3 : 4;
  constexpr int STEPS = 16;                // mma k-steps per item ( = IPT * V / 4 )
  constexpr int NB = 8 * MB;               // padded batch
  extern __shared__ __align__(16) unsigned char smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int J = p.K / V;

  const size_t img_bytes = (static_cast<size_t>(p.C) << (ENTRY_LOG2 + p.rep_log2));
  unsigned char* img = smem;
  float* red = reinterpret_cast<float*>(smem + img_bytes);  // [2][kWarps][NB][kRedStride]
  __shared__ int s_last;

  const uint32_t img_base = smem_u32(img) + ((lane & ((1 << p.rep_log2) - 1)) << ENTRY_LOG2);
  const int entry_shift = ENTRY_LOG2 + p.rep_log2;

  // static contiguous partition of the items, chunk-major so X stays in registers
  const long long items_total = static_cast<long long>(p.nchunks) * p.nrbg;
  const int it_begin = static_cast<int>(items_total * blockIdx.x / gridDim.x);
  const int it_end = static_cast<int>(items_total * (blockIdx.x + 1) / gridDim.x);
  const int n_items = it_end - it_begin;
  if (n_items <= 0) return;

  // warp role inside a chunk: (slice, row lane)
  const int nsl_full = min(kWarps, p.nslices);
  const int wsl = warp % nsl_full;   // slice of this warp inside the chunk
  const int wrl = warp / nsl_full;   // row lane of this warp
  const bool role_ok = wrl < p.rl;

  uint32_t xf[MB][STEPS][2];
  int cur_chunk = -1, cur_group = -1;
  bool active = false;               // this warp has a slice in the current chunk

  IdxRegs<WORDS> ring[kPrefetch][2];

  auto item_coords = [&](int it, int& chunk, int& rbg) {
    chunk = it / p.nrbg;
    rbg = it - chunk * p.nrbg;
  };
  auto issue_loads = [&](int it, IdxRegs<WORDS> (&dst)[2]) {
    int chunk, rbg;
    item_coords(it, chunk, rbg);
    const int slice = chunk * kWarps + wsl;
    if (role_ok && slice < p.nslices) {
      const int row = (rbg * p.rl + wrl) * 16 + g;
      const size_t off = (static_cast<size_t>(row) * J + static_cast<size_t>(slice) * (kSliceK / V) + t4 * IPT) * IB;
      const unsigned char* base = static_cast<const unsigned char*>(p.idx);
      load_idx<WORDS>(dst[0], base + off);
      load_idx<WORDS>(dst[1], base + off + static_cast<size_t>(8) * J * IB);
    }
  };

#pragma unroll
  for (int s = 0; s < kPrefetch - 1; ++s)
    if (s < n_items) issue_loads(it_begin + s, ring[s]);

  for (int it0 = 0; it0 < n_items; it0 += kPrefetch) {
#pragma unroll
    for (int s = 0; s < kPrefetch; ++s) {
      const int li = it0 + s;
      if (li >= n_items) break;
      const int it = it_begin + li;
      if (li + kPrefetch - 1 < n_items) issue_loads(it + kPrefetch - 1, ring[(s + kPrefetch - 1) % kPrefetch]);

      int chunk, rbg;
      item_coords(it, chunk, rbg);
      const int group = (rbg * p.rl * 16) / p.rows_per_cb;

      if (chunk != cur_chunk) {  // (re)load this warp's X fragments: 64 consecutive K values per batch row
        cur_chunk = chunk;
        const int slice = chunk * kWarps + wsl;
        active = role_ok && slice < p.nslices;
        if (active) {
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            const int m = mb * 8 + g;
            const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.K + slice * kSliceK + t4 * 64);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              uint4 vv = make_uint4(0, 0, 0, 0);
              if (m < p.M) vv = __ldg(src + q);
              xf[mb][2 * q][0] = vv.x; xf[mb][2 * q][1] = vv.y;
              xf[mb][2 * q + 1][0] = vv.z; xf[mb][2 * q + 1][1] = vv.w;
            }
          }
        }
      }
      if (group != cur_group) {  // rebuild the replicated codebook image
        __syncthreads();         // everyone is done looking up in the old image
        cur_group = group;
        const int reps = 1 << p.rep_log2;
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.cb) +
                                   (static_cast<size_t>(group) * p.C << ENTRY_LOG2);
        if constexpr (V == 4) {
          if (reps >= 2) {       // one 16-byte store = two replicas of an 8-byte entry
            const int units = (p.C * reps) >> 1;
            for (int u = tid; u < units; u += kThreads) {
              const int c = u / (reps >> 1);
              const uint2 e = __ldg(reinterpret_cast<const uint2*>(src) + c);
              reinterpret_cast<uint4*>(img)[u] = make_uint4(e.x, e.y, e.x, e.y);
            }
          } else {
            for (int u = tid; u < p.C; u += kThreads)
              reinterpret_cast<uint2*>(img)[u] = __ldg(reinterpret_cast<const uint2*>(src) + u);
          }
        } else {
          const int units = p.C * reps;
          for (int u = tid; u < units; u += kThreads)
            reinterpret_cast<uint4*>(img)[u] = __ldg(reinterpret_cast<const uint4*>(src) + (u >> p.rep_log2));
        }
        __syncthreads();
      }

      float acc[MB][4];
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) { acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f; }

      if (active) {
        const IdxRegs<WORDS>& r0 = ring[s][0];
        const IdxRegs<WORDS>& r1 = ring[s][1];
#pragma unroll
        for (int i = 0; i < IPT; ++i) {
          uint32_t c0, c1;
          if constexpr (IB == 1) {
            c0 = (r0.w[i >> 2] >> (8 * (i & 3))) & 0xffu;
            c1 = (r1.w[i >> 2] >> (8 * (i & 3))) & 0xffu;
          } else {
            c0 = (r0.w[i >> 1] >> (16 * (i & 1))) & 0xffffu;
            c1 = (r1.w[i >> 1] >> (16 * (i & 1))) & 0xffffu;
          }
          const uint32_t a_lo = img_base + (c0 << entry_shift);
          const uint32_t a_hi = img_base + (c1 << entry_shift);
          if constexpr (V == 4) {
            uint32_t e0x, e0y, e1x, e1y;
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(e0x), "=r"(e0y) : "r"(a_lo));
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(e1x), "=r"(e1y) : "r"(a_hi));
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) mma_16816(acc[mb], e0x, e1x, e0y, e1y, xf[mb][i][0], xf[mb][i][1]);
          } else {
            uint32_t e0[4], e1[4];
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(e0[0]), "=r"(e0[1]), "=r"(e0[2]), "=r"(e0[3]) : "r"(a_lo));
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(e1[0]), "=r"(e1[1]), "=r"(e1[2]), "=r"(e1[3]) : "r"(a_hi));
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              mma_16816(acc[mb], e0[0], e1[0], e0[1], e1[1], xf[mb][2 * i][0], xf[mb][2 * i][1]);
              mma_16816(acc[mb], e0[2], e1[2], e0[3], e1[3], xf[mb][2 * i + 1][0], xf[mb][2 * i + 1][1]);
            }
          }
        }
      }

      // cross-warp reduction, buffer alternates per item so one barrier per item suffices
      float* rb = red + static_cast<size_t>(li & 1) * (kWarps * NB * kRedStride);
      {
        float* mine = rb + warp * (NB * kRedStride);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int b0 = mb * 8 + 2 * t4;
          mine[b0 * kRedStride + g] = acc[mb][0];
          mine[(b0 + 1) * kRedStride + g] = acc[mb][1];
          mine[b0 * kRedStride + g + 8] = acc[mb][2];
          mine[(b0 + 1) * kRedStride + g + 8] = acc[mb][3];
        }
      }
      __syncthreads();

      const int nsl = min(kWarps, p.nslices - chunk * kWarps);  // slices present in this chunk
      const int outs = p.rl * p.M * 16;
      if (p.nchunks == 1) {
        for (int o = tid; o < outs; o += kThreads) {
          const int r = o & 15, m = (o >> 4) % p.M, lr = (o >> 4) / p.M;
          float sum = 0.f;
          for (int sl = 0; sl < nsl; ++sl) sum += rb[(lr * nsl_full + sl) * (NB * kRedStride) + m * kRedStride + r];
          const int row = (rbg * p.rl + lr) * 16 + r;
          const __half h = __float2half_rn(sum);
          const size_t o_off = static_cast<size_t>(m) * p.ld_y + row;
          p.y[o_off] = h;
          for (int q = 0; q < p.n_peers; ++q) p.peer_y[q][o_off] = h;
        }
      } else {
        for (int o = tid; o < outs; o += kThreads) {
          const int r = o & 15, m = (o >> 4) % p.M, lr = (o >> 4) / p.M;
          float sum = 0.f;
          for (int sl = 0; sl < nsl; ++sl) sum += rb[(lr * nsl_full + sl) * (NB * kRedStride) + m * kRedStride + r];
          const int row = (rbg * p.rl + lr) * 16 + r;
          __stcg(p.ws_partial + (static_cast<size_t>(chunk) * p.M + m) * p.N + row, sum);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          const int old = atomicAdd(p.ws_counter + rbg, 1);
          const int last = (old == p.nchunks - 1);
          if (last) p.ws_counter[rbg] = 0;  // leave the counter zero for the next call
          s_last = last;
        }
        __syncthreads();
        if (s_last) {
          __threadfence();
          for (int o = tid; o < outs; o += kThreads) {
            const int r = o & 15, m = (o >> 4) % p.M, lr = (o >> 4) / p.M;
            const int row = (rbg * p.rl + lr) * 16 + r;
            float sum = 0.f;
            for (int c = 0; c < p.nchunks; ++c)
              sum += __ldcg(p.ws_partial + (static_cast<size_t>(c) * p.M + m) * p.N + row);
            const __half h = __float2half_rn(sum);
            const size_t o_off = static_cast<size_t>(m) * p.ld_y + row;
            p.y[o_off] = h;
            for (int q = 0; q < p.n_peers; ++q) p.peer_y[q][o_off] = h;
          }
        }
      }
    }
  }
}

int pick_rep_log2(int v, int C, size_t budget) {
  int rep = (v == 4) ? 4 : 3;  // 16 or 8 replicas fill a 128-byte line
  while (rep > 0 && (static_cast<size_t>(C) * 2 * v << rep) > budget) --rep;
  return rep;
}

bool fill_params(const Problem& p, DecodeParams& d, size_t& smem_bytes) {
  if (p.M < 1 || p.M > 16) return false;
  if (!(p.v == 4 || p.v == 8)) return false;
  if (!(p.idx_bytes == 1 || p.idx_bytes == 2)) return false;
  if (p.K % kSliceK != 0 || p.N % 16 != 0 || p.K == 0 || p.N == 0) return false;
  const bool single = p.rows_per_cb >= p.N;
  if (!single && p.rows_per_cb % 16 != 0) return false;
  if (p.idx_bytes == 1 && p.C > 256) return false;
  if (p.C > 65536 || p.C < 1) return false;
  if (reinterpret_cast<uintptr_t>(p.x) % 16 || reinterpret_cast<uintptr_t>(p.idx) % 16 ||
      reinterpret_cast<uintptr_t>(p.cb) % 16)
    return false;
  const size_t entry = static_cast<size_t>(2) * p.v;
  if (p.C * entry > 160 * 1024) return false;
  d.nslices = p.K / kSliceK;
  d.nchunks = (d.nslices + kWarps - 1) / kWarps;
  const int nsl_full = d.nslices < kWarps ? d.nslices : kWarps;
  int rl = kWarps / nsl_full;
  const int blocks_per_group = single ? (p.N / 16) : (p.rows_per_cb / 16);
  while (rl > 1 && ((p.N / 16) % rl != 0 || blocks_per_group % rl != 0)) --rl;
  d.rl = rl;
  d.nrbg = p.N / (16 * rl);
  const int MB = p.M <= 8 ? 1 : 2;
  const size_t red_bytes = static_cast<size_t>(2) * kWarps * (8 * MB) * kRedStride * sizeof(float);
  d.rep_log2 = pick_rep_log2(p.v, p.C, 64 * 1024 > p.C * entry ? 64 * 1024 : p.C * entry);
  smem_bytes = (static_cast<size_t>(p.C) * entry << d.rep_log2) + red_bytes;
  if (smem_bytes > 200 * 1024) return false;
  d.x = p.x; d.idx = p.idx; d.cb = p.cb; d.y = p.y;
  d.M = p.M; d.N = p.N; d.K = p.K; d.C = p.C;
  d.rows_per_cb = single ? p.N : p.rows_per_cb;
  d.ld_y = p.ld_y;
  d.n_peers = p.n_peers;
  for (int i = 0; i < 8; ++i) d.peer_y[i] = p.peer_y[i];
  return true;
}

}  // namespace

bool decode_supported(const Problem& p) {
  DecodeParams d{};
  size_t smem;
  return fill_params(p, d, smem);
}

size_t decode_workspace_bytes(const Problem& p) {
  DecodeParams d{};
  size_t smem;
  if (!fill_params(p, d, smem) || d.nchunks == 1) return 0;
  return kCounterBytes + static_cast<size_t>(d.nchunks) * p.M * p.N * sizeof(float);
}

int launch_decode(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s) {
  DecodeParams d{};
  size_t smem;
  if (!fill_params(p, d, smem)) return VQG_ERR_UNSUPPORTED;
  if (d.nchunks > 1) {
    const size_t need = decode_workspace_bytes(p);
    if (ws == nullptr || ws_bytes < need) return VQG_ERR_WORKSPACE;
    if (static_cast<size_t>(d.nrbg) * sizeof(int) > kCounterBytes) return VQG_ERR_UNSUPPORTED;
    d.ws_counter = static_cast<int*>(ws);
    d.ws_partial = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + kCounterBytes);
  }
  d.status = device_status_ptr();

  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long items = static_cast<long long>(d.nchunks) * d.nrbg;
  const int grid = static_cast<int>(items < sms ? items : sms);

  const int MB = p.M <= 8 ? 1 : 2;
  using KernelT = void (*)(const DecodeParams);
  KernelT k = nullptr;
#define VQG_PICK(V_, IB_)                                                   \
  if (p.v == V_ && p.idx_bytes == IB_)                                      \
    k = (MB == 1) ? vq_decode_kernel<V_, IB_, 1> : vq_decode_kernel<V_, IB_, 2>;
  VQG_PICK(4, 1) VQG_PICK(8, 1) VQG_PICK(4, 2) VQG_PICK(8, 2)
#undef VQG_PICK
  if (!k) return VQG_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return VQG_ERR_LAUNCH;
  k<<<grid, kThreads, smem, s>>>(d);
  count_launch();
  return cuda_status(cudaGetLastError());
}


// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the split-K scratch (arrival counters + fp32 partial sums) lives in a
// fixed array inside the library image instead of a caller-provided workspace.  Every GPU that
// loads the library carries these kStaticScratchBytes until the process exits.
//
// `g_static_scratch` below is a device symbol: in host code its name is only a stand-in and must
// not be handed to a kernel.  The device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that pointer is what the kernel receives.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t kStaticScratchBytes = static_cast<size_t>(VQG_NOALLOC_SCRATCH_BYTES);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_static_mu;
unsigned char* g_static_ptr[64] = {};

// Device address of the static scratch on the current device; looked up on the first call per device.
int static_scratch_ptr(unsigned char** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return VQG_ERR_NO_DEVICE;
  if (dev < 0 || dev >= 64) return VQG_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    unsigned char* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) return VQG_ERR_LAUNCH;
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return VQG_OK;
}
}  // namespace

int launch_decode_static(const Problem& p, cudaStream_t s) {
  DecodeParams d{};
  size_t smem;
  if (!fill_params(p, d, smem)) return VQG_ERR_UNSUPPORTED;
  const size_t need = d.nchunks > 1 ? kCounterBytes + static_cast<size_t>(d.nchunks) * p.M * p.N * sizeof(float) : 0;
  if (need > kStaticScratchBytes) return VQG_ERR_TOO_LARGE;
  if (static_cast<size_t>(d.nrbg) * sizeof(int) > kCounterBytes) return VQG_ERR_TOO_LARGE;
  unsigned char* scratch = nullptr;
  const int st = static_scratch_ptr(&scratch);
  if (st != VQG_OK) return st;
  if (d.nchunks > 1) {
    // the array keeps whatever the previous call left: the arrival counters must start at zero
    if (cudaMemsetAsync(scratch, 0, static_cast<size_t>(d.nrbg) * sizeof(int), s) != cudaSuccess) return VQG_ERR_LAUNCH;
    d.ws_counter = reinterpret_cast<int*>(scratch);
    d.ws_partial = reinterpret_cast<float*>(scratch + kCounterBytes);
  }
  d.status = nullptr;

  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long items = static_cast<long long>(d.nchunks) * d.nrbg;
  const int grid = static_cast<int>(items < sms ? items : sms);
  const int MB = p.M <= 8 ? 1 : 2;
  using KernelT = void (*)(const DecodeParams);
  KernelT k = nullptr;
#define VQG_PICK(V_, IB_)                                                   \
  if (p.v == V_ && p.idx_bytes == IB_)                                      \
    k = (MB == 1) ? vq_decode_kernel<V_, IB_, 1> : vq_decode_kernel<V_, IB_, 2>;
  VQG_PICK(4, 1) VQG_PICK(8, 1) VQG_PICK(4, 2) VQG_PICK(8, 2)
#undef VQG_PICK
  if (!k) return VQG_ERR_UNSUPPORTED;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return VQG_ERR_LAUNCH;
  k<<<grid, kThreads, smem, s>>>(d);
  count_launch();
  return cuda_status(cudaGetLastError());
}

}  // namespace vqg
