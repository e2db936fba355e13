// Compute-bound VQ-GEMM for sm_100a, CTA-pair version: two CTAs of a cluster (two SMs) work on one
// 256(M) x 256(N) output tile with tcgen05.mma.cta_group::2.
//
// Why pairs: the single-CTA kernel (tensor.cu) is bound by the shared-memory pipe -- per 64-wide K step
// an SM moves 32 KiB of codebook lookups, 32 KiB of B stores, 48 KiB of UMMA operand reads and 16 KiB of
// TMA writes for 512 cycles of MMA.  In a pair each CTA dequantises only ITS half of B (128 weight rows)
// and the tensor core of each SM reads A (its own 128 rows of X) plus half of B: 16 + 16 + 32 + 16 = 80 KiB
// per step for the same MMA work per SM.
//
// Roles per CTA (320 threads):
//   warp 0      TMA producer: this CTA's X tile [128 x 64] (and, in the dense variant, its W half)
//   warp 1      pair leader (cluster rank 0): issues the MMAs for both CTAs and commits stage-free /
//               accumulator-ready mbarriers in BOTH CTAs.  In the other CTA the same warp forwards
//               "my A and B for stage s are in place" to the leader with a remote mbarrier arrive.
//   warps 2..5  epilogue of this CTA's 128 output rows (tcgen05.ld -> fp16 -> global / peer copies)
//   warps 6..9  dequant: thread r owns weight row n0 + 128*rank + r (see tensor.cu for the scheme)
//
// No TMA load uses cluster multicast; cross-CTA signalling is plain remote mbarrier arrives and
// tcgen05.commit to an explicit shared::cluster address.  Every mbarrier wait is bounded; on expiry the
// kernel records the wait in the device status word, all roles leave their loops, the cluster
// rendezvous at the end is still reached by every thread, tensor memory is released and the kernel
// returns.
#include "tc_ptx.cuh"

namespace vqg {

using namespace tc;

namespace {

constexpr int BM = 128;          // X rows per CTA (256 per pair)
constexpr int BNH = 128;         // weight rows dequantised per CTA (N half)
constexpr int BN = 256;          // output columns per pair tile
constexpr int BK = 64;
constexpr int kThreads = 320;
constexpr int kDequantWarp0 = 6;
constexpr int kDequantThreads = 128;
constexpr uint32_t kABytes = BM * BK * 2;    // 16 KiB
constexpr uint32_t kBBytes = BNH * BK * 2;   // 16 KiB
constexpr uint32_t kImageBytes = 32 * 1024;
constexpr uint32_t kTmemCols = 512;

struct PairParams {
  const unsigned char* idx;  // [N, K/v] uint8
  const __half* cb;          // [G, C, v]
  __half* y;
  int* status;
  int M, N, K, C;
  int rows_per_cb;
  long long ld_y;
  int m_tiles, n_tiles;      // in 256 x 256 pair tiles
  int n_peers;
  __half* peer_y[8];
};

// kind::f16, A = B = fp16, D = fp32, both K-major, M = 256 (pair), N = 256
constexpr uint32_t kIdescPair = (1u << 4) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);

template <int STAGES, bool DENSE>
struct PairSmem {
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kImage = STAGES * kStageBytes;
  static constexpr uint32_t kBars = kImage + (DENSE ? 0 : kImageBytes);
  // full[S], empty[S], acc_full[2], acc_empty[2], dequant rendezvous
  static constexpr uint32_t kTmemSlot = kBars + (2 * STAGES + 5) * 8;
  static constexpr uint32_t kTotal = kTmemSlot + 16;
};

template <int V, bool DENSE, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
vq_tensor_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                      const PairParams p) {
  using L = PairSmem<STAGES, DENSE>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;   // SWIZZLE_128B tiles need 1024-byte alignment
  unsigned char* base_ptr = smem_dyn + (base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();         // 0 = pair leader
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int ksteps = p.K / BK;
  const int total_tiles = p.m_tiles * p.n_tiles;

  auto a_addr = [&](int s) { return base + s * L::kStageBytes; };
  auto b_addr = [&](int s) { return base + s * L::kStageBytes + kABytes; };
  // full[s]: this CTA's TMA bytes have landed (1 arrival + bytes) and, in the fused variant, its 4 dequant
  // warps have written B; in the leader one more arrival says the same of the second CTA.
  auto bar_full = [&](int s) { return base + L::kBars + 8 * s; };
  auto bar_empty = [&](int s) { return base + L::kBars + 8 * (STAGES + s); };
  auto bar_acc_full = [&](int a) { return base + L::kBars + 8 * (2 * STAGES + a); };
  auto bar_acc_empty = [&](int a) { return base + L::kBars + 8 * (2 * STAGES + 2 + a); };
  const uint32_t bar_dq = base + L::kBars + 8 * (2 * STAGES + 4);
  // shared::cluster address of the same offset in the other CTA = local address + a constant
  const uint32_t to_peer = map_to_cta(base, rank ^ 1u) - base;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::kTmemSlot);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1 + (DENSE ? 0 : kDequantThreads / 32) + (rank == 0 ? 1 : 0));
      mbar_init(bar_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_acc_full(a), 1);
      mbar_init(bar_acc_empty(a), 8);   // 4 epilogue warps in each CTA of the pair
    }
    mbar_init(bar_dq, kDequantThreads);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    // both CTAs of the pair allocate together (same warp index, same destination offset)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + L::kTmemSlot),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's mbarriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs) {
        const int m0 = (tile % p.m_tiles) * 256 + static_cast<int>(rank) * BM;
        const int n0 = (tile / p.m_tiles) * BN + static_cast<int>(rank) * BNH;
        for (int kt = 0; kt < ksteps; ++kt) {
          if (!(ok = mbar_wait_cluster(bar_empty(stage), phase ^ 1, p.status, DS_STAGE_EMPTY_TIMEOUT))) break;
          mbar_expect_tx(bar_full(stage), DENSE ? (kABytes + kBBytes) : kABytes);
          tma_load_2d(a_addr(stage), &tmap_x, kt * BK, m0, bar_full(stage));
          if (DENSE) tma_load_2d(b_addr(stage), &tmap_w, kt * BK, n0, bar_full(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (rank == 0) {
        // ------------------------------- MMA issuer (pair leader) ---------------------------
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs) {
          if (!(ok = mbar_wait_cluster(bar_acc_empty(acc), acc_phase ^ 1, p.status, DS_ACC_EMPTY_TIMEOUT))) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
          for (int kt = 0; kt < ksteps; ++kt) {
            if (!(ok = mbar_wait_cluster(bar_full(stage), phase, p.status, DS_TMA_FULL_TIMEOUT))) break;
            tc_fence_after();
            const uint64_t ad = make_desc(a_addr(stage));
            const uint64_t bd = make_desc(b_addr(stage));
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              tc_mma_f16_pair(d_tmem, ad + 2 * k, bd + 2 * k, kIdescPair, (kt | k) != 0 ? 1u : 0u);
            // the stage is free in both CTAs once these MMAs have read it
            tc_commit_pair(bar_empty(stage));
            tc_commit_pair(bar_empty(stage) + to_peer);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          tc_commit_pair(bar_acc_full(acc));
          tc_commit_pair(bar_acc_full(acc) + to_peer);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      } else {
        // ------------------------------- forwarder (second CTA) -----------------------------
        for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs) {
          for (int kt = 0; kt < ksteps; ++kt) {
            if (!(ok = mbar_wait(bar_full(stage), phase, p.status, DS_TMA_FULL_TIMEOUT))) break;
            mbar_arrive_remote(bar_full(stage) + to_peer);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp < kDequantWarp0) {
    // ------------------------------- epilogue -----------------------------------------------
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t leader_acc_empty0 = bar_acc_empty(0) + (rank == 0 ? 0u : to_peer);
    const uint32_t leader_acc_empty1 = bar_acc_empty(1) + (rank == 0 ? 0u : to_peer);
    for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs) {
      const int m0 = (tile % p.m_tiles) * 256 + static_cast<int>(rank) * BM;
      const int n0 = (tile / p.m_tiles) * BN;
      if (!(ok = mbar_wait_cluster(bar_acc_full(acc), acc_phase, p.status, DS_ACC_FULL_TIMEOUT))) break;
      tc_fence_after();
      const int m = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        const int n = n0 + c * 32;
        if (m < p.M && n < p.N) {
          uint4 o[4];
          uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __half2 h = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            ow[i] = *reinterpret_cast<uint32_t*>(&h);
          }
          const size_t off = static_cast<size_t>(m) * p.ld_y + n;
          uint4* dst = reinterpret_cast<uint4*>(p.y + off);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = o[i];
          for (int q = 0; q < p.n_peers; ++q) {
            uint4* pd = reinterpret_cast<uint4*>(p.peer_y[q] + off);
#pragma unroll
            for (int i = 0; i < 4; ++i) pd[i] = o[i];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc == 0 ? leader_acc_empty0 : leader_acc_empty1);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else if (!DENSE) {
    // ------------------------------- dequant warps ------------------------------------------
    constexpr int ENTRY_LOG2 = (V == 4) ? 3 : 4;       // bytes per codebook entry
    constexpr int REPS = 128 >> ENTRY_LOG2;             // replicas filling a 128-byte line
    constexpr int WPS = (BK / V) / 4;                   // index words per K step (uint8 indices)
    constexpr int GSTEPS = 16 / WPS;                    // K steps per 64-byte granule
    const int r = threadIdx.x - kDequantWarp0 * 32;     // B-half row owned by this thread
    const int J = p.K / V;                              // index bytes per weight row
    unsigned char* image = base_ptr + L::kImage;
    const uint32_t img = base + L::kImage + ((lane & (REPS - 1)) << ENTRY_LOG2);
    const uint32_t row_off = static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128);
    const uint32_t rx = static_cast<uint32_t>(r & 7);

    int stage = 0;
    uint32_t phase = 0;
    int cur_group = -1;
    bool ok = true;
    uint32_t dq_phase = 0;
    auto dq_sync = [&]() -> bool {   // bounded rendezvous of the dequant threads of this CTA
      mbar_arrive(bar_dq);
      const bool done = mbar_wait(bar_dq, dq_phase, p.status, DS_DEQUANT_SYNC_TIMEOUT);
      dq_phase ^= 1;
      return done;
    };
    for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs) {
      const int n_half0 = (tile / p.m_tiles) * BN + static_cast<int>(rank) * BNH;
      const int n = n_half0 + r;
      const bool row_valid = n < p.N;
      const int group = (n_half0 < p.N ? n_half0 : p.N - 1) / p.rows_per_cb;
      if (group != cur_group) {
        cur_group = group;
        if (!(ok = dq_sync())) break;   // every thread has finished its lookups in the old image
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.cb) + (static_cast<size_t>(group) * p.C << ENTRY_LOG2);
        if (V == 4) {
          for (int u = r; u < p.C * (REPS / 2); u += kDequantThreads) {
            const uint2 e = __ldg(reinterpret_cast<const uint2*>(src) + u / (REPS / 2));
            reinterpret_cast<uint4*>(image)[u] = make_uint4(e.x, e.y, e.x, e.y);
          }
        } else {
          for (int u = r; u < p.C * REPS; u += kDequantThreads)
            reinterpret_cast<uint4*>(image)[u] = __ldg(reinterpret_cast<const uint4*>(src) + u / REPS);
        }
        if (!(ok = dq_sync())) break;
      }

      const unsigned char* row_ptr = p.idx + static_cast<size_t>(row_valid ? n : 0) * J;
      uint32_t cur[16], nxt[16];
      auto load_granule = [&](int gi, uint32_t (&dst)[16]) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 t = make_uint4(0, 0, 0, 0);
          const int byte0 = gi * 64 + q * 16;
          if (row_valid && byte0 + 16 <= J) t = __ldg(reinterpret_cast<const uint4*>(row_ptr + byte0));
          dst[4 * q] = t.x; dst[4 * q + 1] = t.y; dst[4 * q + 2] = t.z; dst[4 * q + 3] = t.w;
        }
      };
      const int ngran = (ksteps + GSTEPS - 1) / GSTEPS;
      load_granule(0, nxt);
      for (int gi = 0; ok && gi < ngran; ++gi) {
#pragma unroll
        for (int i = 0; i < 16; ++i) cur[i] = nxt[i];
        if (gi + 1 < ngran) load_granule(gi + 1, nxt);
#pragma unroll
        for (int st = 0; st < GSTEPS; ++st) {
          const int kt = gi * GSTEPS + st;
          if (kt >= ksteps) break;
          if (!(ok = mbar_wait_cluster(bar_empty(stage), phase ^ 1, p.status, DS_STAGE_EMPTY_TIMEOUT))) break;
          const uint32_t dst_row = b_addr(stage) + row_off;
          // all lookups of the row first, then the stores: the loads are independent of one another, so the
          // warp is not held up chunk by chunk waiting for shared-memory latency
          // all lookups of the row first, then the stores: the loads are independent of one another, so the
          // warp is not held up chunk by chunk waiting for shared-memory latency
          uint4 ch[8];
          if (V == 4) {
#pragma unroll
            for (int w = 0; w < WPS; ++w) {
              const uint32_t word = cur[st * WPS + w];
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const uint32_t c0 = (word >> (16 * hh)) & 0xffu, c1 = (word >> (16 * hh + 8)) & 0xffu;
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(ch[2 * w + hh].x), "=r"(ch[2 * w + hh].y) : "r"(img + (c0 << 7)));
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(ch[2 * w + hh].z), "=r"(ch[2 * w + hh].w) : "r"(img + (c1 << 7)));
              }
            }
          } else {
#pragma unroll
            for (int w = 0; w < WPS; ++w) {
              const uint32_t word = cur[st * WPS + w];
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const uint32_t c0 = (word >> (8 * b)) & 0xffu;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(ch[4 * w + b].x), "=r"(ch[4 * w + b].y), "=r"(ch[4 * w + b].z), "=r"(ch[4 * w + b].w)
                             : "r"(img + (c0 << 7)));
              }
            }
          }
#pragma unroll
          for (uint32_t chunk = 0; chunk < 8; ++chunk)
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst_row + ((chunk ^ rx) << 4)), "r"(ch[chunk].x),
                         "r"(ch[chunk].y), "r"(ch[chunk].z), "r"(ch[chunk].w)
                         : "memory");
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  }

  // ------------------------------- teardown --------------------------------------------------
  // Nobody leaves before both CTAs are done: the leader's MMAs read the peer's shared memory and
  // both CTAs signal each other's mbarriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeFn>(f);
  }();
  return fn;
}

// fp16 row-major [rows, cols] matrix, box [128 rows x 64 cols], 128-byte swizzle, zero fill.
bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename Kern>
int launch_pair(Kern kernel, size_t smem, const CUtensorMap& mx, const CUtensorMap& mw, PairParams& tp, cudaStream_t s) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return VQG_ERR_LAUNCH;
  // how many CTA pairs can be resident at once (GPCs with an odd number of usable SMs lose one)
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1));
  int max_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg) != cudaSuccess || max_clusters < 1) {
    cudaGetLastError();
    max_clusters = sms / 2;
  }
  const int tiles = tp.m_tiles * tp.n_tiles;
  const int pairs = tiles < max_clusters ? tiles : max_clusters;
  kernel<<<2 * pairs, kThreads, smem, s>>>(mx, mw, tp);
  count_launch();
  return cuda_status(cudaGetLastError());
}

bool pair_shape_ok(int M, int N, int K, const void* x, const void* y, long long ld_y) {
  if (M < 1 || N < 1 || K < BK || K % BK != 0) return false;
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(y) % 16) return false;
  if (N % 32 != 0 || ld_y % 8 != 0) return false;
  return true;
}

}  // namespace

bool tensor_pair_supported(const Problem& p) {
  if (!pair_shape_ok(p.M, p.N, p.K, p.x, p.y, p.ld_y)) return false;
  if (!(p.v == 4 || p.v == 8) || p.idx_bytes != 1 || p.C < 1 || p.C > 256) return false;
  if ((p.K / p.v) % 16 != 0) return false;  // 16-byte index loads per row
  if (reinterpret_cast<uintptr_t>(p.idx) % 16 || reinterpret_cast<uintptr_t>(p.cb) % 16) return false;
  const bool single = p.rows_per_cb >= p.N;
  if (!single && p.rows_per_cb % 128 != 0) return false;
  return true;
}

int launch_tensor_pair(const Problem& p, cudaStream_t s) {
  if (!tensor_pair_supported(p)) return VQG_ERR_UNSUPPORTED;
  CUtensorMap mx;
  if (!make_map(&mx, p.x, p.M, p.K)) return VQG_ERR_LAUNCH;
  PairParams tp{};
  tp.idx = static_cast<const unsigned char*>(p.idx);
  tp.cb = p.cb;
  tp.y = p.y;
  tp.status = device_status_ptr();
  tp.M = p.M; tp.N = p.N; tp.K = p.K; tp.C = p.C;
  tp.rows_per_cb = p.rows_per_cb >= p.N ? p.N : p.rows_per_cb;
  tp.ld_y = p.ld_y;
  tp.m_tiles = (p.M + 255) / 256;
  tp.n_tiles = (p.N + BN - 1) / BN;
  tp.n_peers = p.n_peers;
  for (int i = 0; i < 8; ++i) tp.peer_y[i] = p.peer_y[i];
  constexpr int S = 5;
  const size_t smem = PairSmem<S, false>::kTotal + 1024;
  if (p.v == 4) return launch_pair(vq_tensor_pair_kernel<4, false, S>, smem, mx, mx, tp, s);
  return launch_pair(vq_tensor_pair_kernel<8, false, S>, smem, mx, mx, tp, s);
}

int launch_dense_pair(const __half* x, const __half* w_nk, __half* y, int M, int N, int K, long long ld_y, int n_peers,
                      __half* const* peer_y, cudaStream_t s) {
  if (!pair_shape_ok(M, N, K, x, y, ld_y) || reinterpret_cast<uintptr_t>(w_nk) % 16) return VQG_ERR_UNSUPPORTED;
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K) || !make_map(&mw, w_nk, N, K)) return VQG_ERR_LAUNCH;
  PairParams tp{};
  tp.y = y;
  tp.status = device_status_ptr();
  tp.M = M; tp.N = N; tp.K = K; tp.C = 0;
  tp.rows_per_cb = N;
  tp.ld_y = ld_y;
  tp.m_tiles = (M + 255) / 256;
  tp.n_tiles = (N + BN - 1) / BN;
  tp.n_peers = n_peers;
  for (int i = 0; i < n_peers && i < 8; ++i) tp.peer_y[i] = peer_y[i];
  constexpr int S = 6;
  const size_t smem = PairSmem<S, true>::kTotal + 1024;
  return launch_pair(vq_tensor_pair_kernel<4, true, S>, smem, mx, mw, tp, s);
}

}  // namespace vqg
