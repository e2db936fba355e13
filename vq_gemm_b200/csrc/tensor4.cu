// Small-batch VQ-GEMM (M <= 128) for sm_100a with the dequantised weights as the MMA's TENSOR-MEMORY
// operand and a work-balanced (stream-K) split of the K loop.
//
//     D^T[n, m] = sum_k W[n, k] * X[m, k]      MMA M = 128 weight rows (one CTA), N = NB batch columns
//
// At small M the product is a stream over the index matrix: what limits it is one shared-memory codebook
// lookup per index and fixed per-CTA costs, not flops.  This kernel keeps the tensor core for the
// arithmetic (no fragment registers for X, no cross-warp reduction: the accumulator sits in TMEM for the
// whole K range of a CTA) and spends its threads on lookups:
//
//   warp 0       TMA producer: X tile [NB x 128 K values] (rows >= M are zero-filled)
//   warps 1..4   MMA issue (one lane each): a tcgen05.mma of 128 x NB x 16 is almost no work for the tensor
//                core at small NB, so the cadence at which ONE thread can issue them (~65 cycles each)
//                would bound the kernel; 4 (NB <= 64) or 2 warps each issue a share of a stage's 8 MMAs
//                into their own accumulator, and the epilogue adds the accumulators in a fixed order
//   warps 5..8   epilogue: tcgen05.ld of D^T (lane = weight row); a CTA that covered the whole K range of
//                a tile writes Y directly, otherwise it writes fp32 partials to the workspace and the
//                last-arriving contributor of that tile (per 32-row quarter) sums them in contributor
//                order -- deterministic
//   warps 9..24  dequant: 4 warps per TMEM lane quarter; thread = weight row; warp j of a quarter takes
//                every 4th 64-wide K sub-step: 16-byte index load, lookups in the (replicated,
//                conflict-free when C <= 256) codebook image, one tcgen05.st of 32 columns
//
// Work split: the (128-row tile, K stage) pairs (a stage is 128 K values, 256 on large matrices) are numbered
// tile-major and divided evenly over
// the CTAs, so every SM gets the same number of stages whatever N and K are; a CTA's range touches one
// to a few tiles ("segments").  Every mbarrier wait is bounded (see tensor2.cu).
//
// There is no reference counterpart: the reference requires M % 128 == 0 (strategy_1/src.cu:221).
#include "tc_ptx.cuh"

namespace vqg {

using namespace tc;

namespace {

constexpr int BNROWS = 128;      // weight rows per tile (TMEM lanes)
constexpr int BK = 64;           // K values per sub-step
constexpr int kThreads = 800;    // 25 warps
constexpr int kMmaWarps = 4;     // MMA-issuing warps (one lane each), each with its own accumulator
constexpr int kEpiWarp0 = 1 + kMmaWarps;
constexpr int kDequantWarp0 = kEpiWarp0 + 4;
constexpr int kDequantWarps = 16;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAColsPerSub = BK / 2;             // 32 columns: two fp16 per 32-bit column

struct SmallParams {
  const unsigned char* idx;
  const __half* cb;
  __half* y;
  float* ws_partial;   // [tile][slot][M][128]
  int* ws_counter;     // [tile][4]
  int* status;
  int M, N, K, C;
  int rows_per_cb;
  long long ld_y;
  int ntiles, ksteps;  // tiles of 128 weight rows; 128-wide K stages per tile
  int q, r;            // stages per CTA: q, one more for the first r CTAs
  int max_slots;
  int n_peers;
  __half* peer_y[8];
};

// The X tiles are tiny at small M (4 KiB per stage for 16 batch columns) but every TMA load still takes
// about a microsecond, far longer than the ~256 cycles a stage of lookups needs: X gets its own, deeper
// ring (up to 16 stages) so that the loads run well ahead of the 4-stage tensor-memory ring of A.
// KS: 64-wide sub-steps per pipeline stage.  2 by default; 4 (256-wide stages, half the hand-overs per K) for
// matrices large enough that every CTA still gets many stages -- measured 14 % faster there, slower elsewhere.
template <int NB, int KS>
struct SmallSmem {
  static constexpr uint32_t kXSub = NB * BK * 2;                 // one 64-wide sub-tile of X
  static constexpr uint32_t kXStage = KS * kXSub;
  static constexpr uint32_t kXSubAligned = (kXSub + 1023u) & ~1023u;
  static constexpr uint32_t kXStageAligned = KS * kXSubAligned;
  static constexpr int kXStages = (NB <= 16 ? 16 : (NB <= 32 ? 12 : (NB <= 64 ? 6 : 4))) * 2 / KS;
  static constexpr uint32_t kImage = kXStages * kXStageAligned;
  // A stages in tensor memory: what the 512 columns leave after the accumulators (4 x NB columns up to 64
  // batch columns, 2 x 128 above).  Measured: 7 stages are no faster than 4, and 2 issuing warps no slower
  // than 4 -- neither the ring depth nor the issue rate of one thread bounds this kernel
  static constexpr int kStages = KS == 2 ? (NB <= 16 ? 7 : (NB <= 32 ? 6 : 4)) : (NB <= 32 ? 3 : 2);
  static constexpr int kBarriers = 2 * kXStages + 2 * kStages + 3;
};

__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// first stage of CTA b, and the CTA that owns stage s, for the even split (q, r)
__device__ __forceinline__ int cta_begin(int b, int q, int r) { return b * q + min(b, r); }
__device__ __forceinline__ int cta_of_stage(int s, int q, int r) {
  const int big = r * (q + 1);
  return s < big ? s / (q + 1) : r + (s - big) / q;
}

// V: sub-vector length; IB: index bytes (12: two 12-bit indices packed in three bytes); NB: batch columns of the MMA
// (16..128); REPL: replicated image.
template <int V, int IB, int NB, bool REPL, int KS>
__global__ void __launch_bounds__(kThreads, 1)
vq_small_ts_kernel(const __grid_constant__ CUtensorMap tmap_x, const SmallParams p) {
  using L = SmallSmem<NB, KS>;
  constexpr uint32_t kAColsPerStage = KS * kAColsPerSub;
  constexpr int ENTRY_LOG2 = (V == 4) ? 3 : 4;
  constexpr int REP_LOG2 = REPL ? (7 - ENTRY_LOG2) : 0;
  constexpr int ENTRY_SHIFT = ENTRY_LOG2 + REP_LOG2;
  constexpr int BPS = IB == 12 ? (BK / V) * 3 / 2 : (BK / V) * IB;   // index bytes per row and sub-step: 16, 8, 16 or 12
  constexpr int WPS = BPS / 4;                          // 32-bit words of indices per sub-step
  // kind::f16, A = B = fp16, D = fp32, both K-major, M = 128, N = NB
  constexpr uint32_t kIdesc = (1u << 4) | (static_cast<uint32_t>(NB >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bid = blockIdx.x;
  // the next kernel in the stream may be scheduled as soon as SMs free up; like this one it waits
  // (griddepcontrol.wait in the TMA and epilogue roles) before it touches X, Y or the workspace
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int s_begin = cta_begin(bid, p.q, p.r);
  const int s_end = cta_begin(bid + 1, p.q, p.r);
  const uint32_t img_bytes = static_cast<uint32_t>(p.C) << ENTRY_SHIFT;
  const uint32_t bars = base + L::kImage + ((img_bytes + 15u) & ~15u);

  auto x_addr = [&](int s, int u) { return base + s * L::kXStageAligned + u * L::kXSubAligned; };
  constexpr int XS = L::kXStages;
  constexpr int STAGES = L::kStages;
  constexpr uint32_t kACols = STAGES * kAColsPerStage;   // the accumulators follow
  constexpr int NW = (NB <= 64) ? kMmaWarps : 2;          // MMA-issuing warps in use, one accumulator each
  constexpr int MPW = (KS * BK / 16) / NW;                 // MMAs per warp and stage
  static_assert(kACols + NW * NB <= kTmemCols, "accumulators do not fit tensor memory");
  // full[s]: one arrival per dequant warp that wrote a quarter of a sub-step of A stage s (8)
  auto bar_full = [&](int s) { return bars + 8 * s; };
  auto bar_empty = [&](int s) { return bars + 8 * (STAGES + s); };
  auto bar_x_full = [&](int s) { return bars + 8 * (2 * STAGES + s); };
  auto bar_x_empty = [&](int s) { return bars + 8 * (2 * STAGES + XS + s); };
  const uint32_t bar_acc_full = bars + 8 * (2 * STAGES + 2 * XS);
  const uint32_t bar_acc_empty = bars + 8 * (2 * STAGES + 2 * XS + 1);
  const uint32_t bar_dq = bars + 8 * (2 * STAGES + 2 * XS + 2);
  const uint32_t tmem_slot_addr = bars + 8 * (2 * STAGES + 2 * XS + 3);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + (tmem_slot_addr - base));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 4 * KS);
      mbar_init(bar_empty(s), NW);
    }
    for (int s = 0; s < XS; ++s) {
      mbar_init(bar_x_full(s), 1);
      mbar_init(bar_x_empty(s), NW);
    }
    mbar_init(bar_acc_full, NW);
    mbar_init(bar_acc_empty, 4);
    mbar_init(bar_dq, kDequantWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot_addr), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t d_tmem = tmem_base + kACols;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      bool ok = true;
      int seq = 0;
      asm volatile("griddepcontrol.wait;" ::: "memory");   // X is the predecessor's to write
      for (int s = s_begin; ok && s < s_end; ++s, ++seq) {
        const int stage = seq % XS;
        const uint32_t phase = (seq / XS) & 1;
        const int kt = s % p.ksteps;
        if (!(ok = mbar_wait(bar_x_empty(stage), phase ^ 1, p.status, DS_STAGE_EMPTY_TIMEOUT))) break;
        mbar_expect_tx(bar_x_full(stage), L::kXStage);
#pragma unroll
        for (int u = 0; u < KS; ++u) tma_load_2d(x_addr(stage, u), &tmap_x, (kt * KS + u) * BK, 0, bar_x_full(stage));
      }
    }
  } else if (warp < kEpiWarp0) {
    // ------------------------------- MMA issuers --------------------------------------------
    const int mw = warp - 1;
    if (lane == 0 && mw < NW) {
      bool ok = true;
      int seq = 0;
      uint32_t acc_phase = 0;
      int s = s_begin;
      const uint32_t d_mine = d_tmem + static_cast<uint32_t>(mw * NB);
      while (ok && s < s_end) {
        const int tile = s / p.ksteps;
        const int seg_end = min(s_end, (tile + 1) * p.ksteps);
        if (!(ok = mbar_wait(bar_acc_empty, acc_phase ^ 1, p.status, DS_ACC_EMPTY_TIMEOUT))) break;
        tc_fence_after();
        for (int first = 1; s < seg_end; ++s, ++seq, first = 0) {
          const int stage = seq % STAGES, xstage = seq % XS;
          const uint32_t phase = (seq / STAGES) & 1, xphase = (seq / XS) & 1;
          if (!(ok = mbar_wait(bar_x_full(xstage), xphase, p.status, DS_TMA_FULL_TIMEOUT))) break;
          if (!(ok = mbar_wait(bar_full(stage), phase, p.status, DS_B_READY_TIMEOUT))) break;
          tc_fence_after();
          const uint32_t a_t = tmem_base + static_cast<uint32_t>(stage) * kAColsPerStage;
#pragma unroll
          for (int i = 0; i < MPW; ++i) {
            const int kk = mw * MPW + i;                  // 16-wide K slice of the stage: sub-tile kk/4, slice kk%4
            const uint64_t bd = make_desc(x_addr(xstage, kk >> 2)) + 2 * (kk & 3);
            tc_mma_f16_ts(d_mine, a_t + 8 * kk, bd, kIdesc, (first && i == 0) ? 0u : 1u);
          }
          tc_commit(bar_empty(stage));
          tc_commit(bar_x_empty(xstage));
        }
        if (!ok) break;
        tc_commit(bar_acc_full);
        acc_phase ^= 1;
      }
    }
  } else if (warp < kDequantWarp0) {
    // ------------------------------- epilogue -----------------------------------------------
    const int quarter = warp & 3;
    uint32_t acc_phase = 0;
    bool ok = true;
    int s = s_begin;
    asm volatile("griddepcontrol.wait;" ::: "memory");     // Y and the workspace follow the stream's order
    while (ok && s < s_end) {
      const int tile = s / p.ksteps;
      const int t0 = tile * p.ksteps;
      const int seg_end = min(s_end, t0 + p.ksteps);
      const bool whole = (s == t0) && (seg_end == t0 + p.ksteps);
      if (!(ok = mbar_wait(bar_acc_full, acc_phase, p.status, DS_ACC_FULL_TIMEOUT))) break;
      tc_fence_after();
      const int row = tile * BNROWS + quarter * 32 + lane;       // weight row = output column
      const uint32_t t_row = d_tmem + (static_cast<uint32_t>(quarter * 32) << 16);
      const int b_first = cta_of_stage(t0, p.q, p.r);
      const int slot = bid - b_first;
      float* part = p.ws_partial + ((static_cast<size_t>(tile) * p.max_slots + slot) * p.M) * BNROWS + quarter * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < NB / 16; ++c) {
        if (c * 16 >= p.M) break;
        uint32_t r[16];
        tmem_ld16(t_row + c * 16, r);
#pragma unroll
        for (int w2 = 1; w2 < NW; ++w2) {             // add the other issuers' accumulators, in order
          uint32_t r2[16];
          tmem_ld16(t_row + w2 * NB + c * 16, r2);
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = c * 16 + j;
          if (m < p.M) {
            if (whole) {
              const __half h = __float2half_rn(__uint_as_float(r[j]));
              const size_t off = static_cast<size_t>(m) * p.ld_y + row;
              p.y[off] = h;
              for (int qq = 0; qq < p.n_peers; ++qq) p.peer_y[qq][off] = h;
            } else {
              __stcg(part + static_cast<size_t>(m) * BNROWS, __uint_as_float(r[j]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty);
      acc_phase ^= 1;
      if (!whole) {
        // the contributor that brings this quarter's counter to the number of contributors sums them in order
        const int b_last = cta_of_stage(t0 + p.ksteps - 1, p.q, p.r);
        const int n_contrib = b_last - b_first + 1;
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          int* ctr = p.ws_counter + tile * 4 + quarter;
          const int old = atomicAdd(ctr, 1);
          last = (old == n_contrib - 1);
          if (last) *ctr = 0;            // leave the counter zero for the next call
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          const float* src = p.ws_partial + (static_cast<size_t>(tile) * p.max_slots * p.M) * BNROWS + quarter * 32 + lane;
          // 16 batch rows at a time with all loads of a contributor in flight together (a serial chain of
          // dependent L2 loads would cost ~700 cycles each); contributors are added in order
          for (int mb = 0; mb < p.M; mb += 16) {
            float sum[16];
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) sum[jj] = 0.f;
            for (int c = 0; c < n_contrib; ++c) {
              float v[16];
#pragma unroll
              for (int jj = 0; jj < 16; ++jj)
                v[jj] = (mb + jj < p.M) ? __ldcg(src + (static_cast<size_t>(c) * p.M + mb + jj) * BNROWS) : 0.f;
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) sum[jj] += v[jj];
            }
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
              if (mb + jj < p.M) {
                const __half h = __float2half_rn(sum[jj]);
                const size_t off = static_cast<size_t>(mb + jj) * p.ld_y + row;
                p.y[off] = h;
                for (int qq = 0; qq < p.n_peers; ++qq) p.peer_y[qq][off] = h;
              }
            }
          }
        }
      }
      s = seg_end;
    }
  } else {
    // ------------------------------- dequant warps ------------------------------------------
    const int dw = warp - kDequantWarp0;          // 0..15
    const int quarter = warp & 3;                  // TMEM lane quarter of this warp
    const int j = dw >> 2;                         // this warp takes sub-steps j, j+4, j+8, ... of the CTA's sequence
    const int rrow = quarter * 32 + lane;          // weight row inside the tile = TMEM lane
    const int tix = dw * 32 + lane;                // 0..511 for cooperative copies
    const size_t J = IB == 12 ? static_cast<size_t>(p.K / V) * 3 / 2 : static_cast<size_t>(p.K / V) * IB;   // index bytes per weight row
    unsigned char* image = base_ptr + L::kImage;
    const uint32_t img = base + L::kImage + ((lane & ((1 << REP_LOG2) - 1)) << ENTRY_LOG2);
    const uint32_t a_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

    bool ok = true;
    uint32_t dq_phase = 0;
    auto dq_sync = [&]() -> bool {   // bounded rendezvous of the 16 dequant warps
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dq);
      const bool done = mbar_wait(bar_dq, dq_phase, p.status, DS_DEQUANT_SYNC_TIMEOUT);
      dq_phase ^= 1;
      return done;
    };
    int cur_group = -1;
    int sub_seq = 0;                               // sub-steps of this CTA before the current segment
    int s = s_begin;
    while (ok && s < s_end) {
      const int tile = s / p.ksteps;
      const int t0 = tile * p.ksteps;
      const int seg_end = min(s_end, t0 + p.ksteps);
      const int nsub = (seg_end - s) * KS;         // sub-steps in this segment
      const int ks0 = (s - t0) * KS;               // first sub-step (within the tile) of the segment
      const int group = (tile * BNROWS) / p.rows_per_cb;
      if (group != cur_group) {
        cur_group = group;
        if (!(ok = dq_sync())) break;              // all lookups in the old image are done
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.cb) + (static_cast<size_t>(group) * p.C << ENTRY_LOG2);
        if constexpr (V == 4) {
          constexpr int HALF_REPS = (1 << REP_LOG2) / 2;
          for (int u = tix; u < p.C * HALF_REPS; u += kDequantWarps * 32) {
            const uint2 e = __ldg(reinterpret_cast<const uint2*>(src) + u / HALF_REPS);
            reinterpret_cast<uint4*>(image)[u] = make_uint4(e.x, e.y, e.x, e.y);
          }
        } else {
          for (int u = tix; u < (p.C << REP_LOG2); u += kDequantWarps * 32)
            reinterpret_cast<uint4*>(image)[u] = __ldg(reinterpret_cast<const uint4*>(src) + (u >> REP_LOG2));
        }
        if (!(ok = dq_sync())) break;
      }
      const unsigned char* row_ptr = p.idx + static_cast<size_t>(tile * BNROWS + rrow) * J;
      // this warp's sub-steps of the segment: local index t = t_first, t_first + 4, ...
      const int t_first = ((j - sub_seq) % 4 + 4) % 4;
      constexpr int PF = 4;                         // index loads in flight per thread
      uint32_t ring[PF][WPS];
      auto load_sub = [&](int t, uint32_t (&dst)[WPS]) {
        if (t < nsub) {
          const unsigned char* src = row_ptr + static_cast<size_t>(ks0 + t) * BPS;
          if constexpr (WPS == 4) {
            const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src));
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
          } else if constexpr (WPS == 3) {               // packed: 12 bytes at a multiple of 4 (rows are multiples of 24 bytes)
            const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src);
            // position inside an aligned 16-byte chunk (the same for every lane when K is a multiple of 256); the
            // 16-byte load at position 0 reads 4 bytes past the 12 and is not used on a row's last sub-step
            const uint32_t in16 = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15);
            if (in16 == 0 && (ks0 + t + 1) * BK < p.K) {                // inside one aligned chunk: one load
              const uint4 q = __ldcs(reinterpret_cast<const uint4*>(src));
              dst[0] = q.x; dst[1] = q.y; dst[2] = q.z;
            } else if (in16 == 4) {
              const uint4 q = __ldcs(reinterpret_cast<const uint4*>(src - 4));
              dst[0] = q.y; dst[1] = q.z; dst[2] = q.w;
            } else if ((in16 & 4) == 0) {                               // 8 + 4 bytes
              const uint2 lo = __ldcs(reinterpret_cast<const uint2*>(src));
              dst[0] = lo.x; dst[1] = lo.y; dst[2] = __ldcs(s32 + 2);
            } else {                                                    // 4 + 8 bytes
              const uint2 hi = __ldcs(reinterpret_cast<const uint2*>(src + 4));
              dst[0] = __ldcs(s32); dst[1] = hi.x; dst[2] = hi.y;
            }
          } else {
            const uint2 v = __ldcs(reinterpret_cast<const uint2*>(src));
            dst[0] = v.x; dst[1] = v.y;
          }
        }
      };
#pragma unroll
      for (int i = 0; i < PF - 1; ++i) load_sub(t_first + 4 * i, ring[i]);
      for (int t0i = 0; ok; t0i += PF) {
        if (t_first + 4 * t0i >= nsub) break;
#pragma unroll
        for (int i = 0; i < PF; ++i) {
          const int t = t_first + 4 * (t0i + i);
          if (t >= nsub) break;
          load_sub(t + 4 * (PF - 1), ring[(i + PF - 1) % PF]);
          const uint32_t* w = ring[i];
          uint32_t a[32];
          if constexpr (V == 4) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const uint32_t c0 = (w[e >> 2] >> (8 * (e & 3))) & 0xffu;
              asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(a[2 * e]), "=r"(a[2 * e + 1]) : "r"(img + (c0 << ENTRY_SHIFT)));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              uint32_t c0;
              if constexpr (IB == 1) {
                c0 = (w[e >> 2] >> (8 * (e & 3))) & 0xffu;
              } else if constexpr (IB == 2) {   // held below C: a larger index (malformed input) would address past the image
                c0 = min((w[e >> 1] >> (16 * (e & 1))) & 0xffffu, static_cast<uint32_t>(p.C - 1));
              } else {                                    // index e sits at bit 12 e of the 96 bits
                constexpr int kNoWord = WPS - 1;
                const int word = (12 * e) >> 5, sh = (12 * e) & 31;
                const uint32_t hi = word < kNoWord ? w[word + 1] : 0u;
                c0 = __funnelshift_r(w[word], hi, sh) & 0xfffu;
                if (p.C < 4096) c0 = c0 < static_cast<uint32_t>(p.C) ? c0 : 0u;   // 12 bits can name more entries than the image holds
              }
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(a[4 * e]), "=r"(a[4 * e + 1]), "=r"(a[4 * e + 2]), "=r"(a[4 * e + 3])
                           : "r"(img + (c0 << ENTRY_SHIFT)));
            }
          }
          const int sseq = sub_seq + t;              // sub-step number in the CTA's sequence
          const int stage_seq = sseq / KS, u = sseq % KS;
          const int stage = stage_seq % STAGES;
          const uint32_t phase = (stage_seq / STAGES) & 1;
          if (!(ok = mbar_wait(bar_empty(stage), phase ^ 1, p.status, DS_STAGE_EMPTY_TIMEOUT))) break;
          tc_fence_after();
          tmem_st32(a_lane + static_cast<uint32_t>(stage) * kAColsPerStage + u * kAColsPerSub, a);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full(stage));
        }
      }
      sub_seq += nsub;
      s = seg_end;
    }
  }

  // ------------------------------- teardown --------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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

bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

struct Plan { int ntiles, ksteps, grid, q, r, max_slots; bool repl; int nb; int ks; };

bool make_plan(const Problem& p, Plan& pl) {
  if (p.M < 1 || p.M > 128 || p.N < 1 || p.K < 128) return false;
  if (p.K % 128 != 0 || p.N % 128 != 0) return false;
  const bool combo = (p.v == 4 && p.idx_bytes == 1) || (p.v == 8 && p.idx_bytes == 1) || (p.v == 8 && p.idx_bytes == 2) ||
                     (p.v == 8 && p.idx_bytes == VQG_IDX_PACKED12);
  if (!combo) return false;
  if (p.idx_bytes == 1 && p.C > 256) return false;
  if (p.C < 1 || p.C > 4096) return false;
  const bool single = p.rows_per_cb >= p.N;
  if (!single && p.rows_per_cb % 128 != 0) return false;
  if (reinterpret_cast<uintptr_t>(p.x) % 16 || reinterpret_cast<uintptr_t>(p.idx) % 16 ||
      reinterpret_cast<uintptr_t>(p.cb) % 16)
    return false;
  pl.repl = p.C <= 256 && p.idx_bytes != VQG_IDX_PACKED12;   // packed indices: one instance, unreplicated image
  if (!pl.repl && p.v != 8) return false;       // large codebooks only with 16-byte entries (64 KiB image)
  pl.nb = p.M <= 16 ? 16 : (p.M <= 32 ? 32 : (p.M <= 64 ? 64 : 128));
  pl.ntiles = p.N / 128;
  const int sms = sm_count();
  // 256-wide stages where a CTA still gets at least 16 of them (replicated codebooks only)
  pl.ks = (pl.repl && p.K % 256 == 0 && static_cast<long long>(pl.ntiles) * (p.K / 256) >= 16LL * sms) ? 4 : 2;
  pl.ksteps = p.K / (pl.ks * BK);
  const long long total = static_cast<long long>(pl.ntiles) * pl.ksteps;
  if (total > (1 << 30)) return false;
  pl.grid = static_cast<int>(total < sms ? total : sms);
  pl.q = static_cast<int>(total / pl.grid);
  pl.r = static_cast<int>(total % pl.grid);
  pl.max_slots = (pl.ksteps + pl.q - 1) / pl.q + 1;
  if (static_cast<size_t>(pl.ntiles) * 4 * sizeof(int) > kCounterBytes) return false;
  return true;
}

}  // namespace

bool small_ts_supported(const Problem& p) {
  Plan pl;
  return make_plan(p, pl);
}

size_t small_ts_workspace_bytes(const Problem& p) {
  Plan pl;
  if (!make_plan(p, pl)) return 0;
  return kCounterBytes + static_cast<size_t>(pl.ntiles) * pl.max_slots * p.M * 128 * sizeof(float);
}

int launch_small_ts(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s) {
  Plan pl;
  if (!make_plan(p, pl)) return VQG_ERR_UNSUPPORTED;
  if (!ws || ws_bytes < small_ts_workspace_bytes(p)) return VQG_ERR_WORKSPACE;
  CUtensorMap mx;
  if (!make_map(&mx, p.x, p.M, p.K, pl.nb)) return VQG_ERR_LAUNCH;
  SmallParams sp{};
  sp.idx = static_cast<const unsigned char*>(p.idx);
  sp.cb = p.cb;
  sp.y = p.y;
  sp.ws_counter = static_cast<int*>(ws);
  sp.ws_partial = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + kCounterBytes);
  sp.status = device_status_ptr();
  sp.M = p.M; sp.N = p.N; sp.K = p.K; sp.C = p.C;
  sp.rows_per_cb = p.rows_per_cb >= p.N ? p.N : p.rows_per_cb;
  sp.ld_y = p.ld_y;
  sp.ntiles = pl.ntiles; sp.ksteps = pl.ksteps; sp.q = pl.q; sp.r = pl.r; sp.max_slots = pl.max_slots;
  sp.n_peers = p.n_peers;
  for (int i = 0; i < 8; ++i) sp.peer_y[i] = p.peer_y[i];

  const size_t entry = static_cast<size_t>(2) * p.v;
  const size_t img = pl.repl ? static_cast<size_t>(p.C) * 128 : static_cast<size_t>(p.C) * entry;
  const bool dependent = !take_weights_written(s);   // not beside a kernel of this library that wrote the weights
  auto launch = [&](auto kernel, size_t x_bytes, int n_bars) -> int {
    size_t smem = x_bytes + ((img + 15) & ~static_cast<size_t>(15)) + (n_bars + 1) * 8 + 16 + 1024;
    // an 8-bit index beyond a small codebook (malformed input) must still address inside the block's shared memory
    if (p.idx_bytes == 1 && p.C < 256 && smem < x_bytes + (img / p.C) * 256 + 1024) smem = x_bytes + (img / p.C) * 256 + 1024;
    if (smem > 227 * 1024) return VQG_ERR_UNSUPPORTED;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return VQG_ERR_LAUNCH;
    // programmatic dependent launch: set-up, codebook image and index prefetch overlap the tail of the
    // kernel before this one in the stream; the roles that touch X, Y or the workspace wait inside
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(pl.grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mx, sp);
    count_launch();
    return cuda_status(e == cudaSuccess ? cudaGetLastError() : e);
  };
#define VQG_SMALL(V_, IB_, NB_, R_, KS_) \
  launch(vq_small_ts_kernel<V_, IB_, NB_, R_, KS_>, SmallSmem<NB_, KS_>::kImage, SmallSmem<NB_, KS_>::kBarriers)
#define VQG_SMALL_NB(V_, IB_, R_, KS_)                                                           \
  (pl.nb == 16 ? VQG_SMALL(V_, IB_, 16, R_, KS_) : pl.nb == 32 ? VQG_SMALL(V_, IB_, 32, R_, KS_) \
   : pl.nb == 64 ? VQG_SMALL(V_, IB_, 64, R_, KS_) : VQG_SMALL(V_, IB_, 128, R_, KS_))
  if (pl.ks == 4) {   // replicated codebooks only
    if (p.v == 4) return VQG_SMALL_NB(4, 1, true, 4);
    if (p.idx_bytes == 1) return VQG_SMALL_NB(8, 1, true, 4);
    return VQG_SMALL_NB(8, 2, true, 4);
  }
  if (p.idx_bytes == VQG_IDX_PACKED12) return VQG_SMALL_NB(8, 12, false, 2);
  if (p.v == 4) return VQG_SMALL_NB(4, 1, true, 2);
  if (p.idx_bytes == 1) return VQG_SMALL_NB(8, 1, true, 2);
  return pl.repl ? VQG_SMALL_NB(8, 2, true, 2) : VQG_SMALL_NB(8, 2, false, 2);
#undef VQG_SMALL_NB
#undef VQG_SMALL
}

}  // namespace vqg
