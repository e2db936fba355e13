// Compute-bound VQ-GEMM for sm_100a with the dequantised weights fed to the tensor core THROUGH TENSOR
// MEMORY (tcgen05.mma with the A operand in TMEM), on CTA pairs (cta_group::2).
//
// Why: with B dequantised into shared memory (tensor.cu, tensor2.cu) every weight byte crosses the
// shared-memory pipe three times (codebook lookup, store into the operand tile, UMMA read) and the
// kernel is bound by that pipe, not by the tensor core.  Here the problem is transposed: the MMA's M
// dimension is the WEIGHT rows and its N dimension the batch rows,
//
//     D^T[n, m] = sum_k W[n, k] * X[m, k]        A = W (from tensor memory), B = X (from shared memory)
//
// A dequant thread owns weight row n = TMEM lane; the 32 registers it looks up per 64-wide K step are
// exactly the 32 tensor-memory columns of its A row (two fp16 per column), written with one tcgen05.st.
// Per K step a CTA's shared-memory pipe then carries only 16 KiB of lookups, 16 KiB of TMA writes (its
// half of the X tile) and 16 KiB of UMMA reads: 48 KiB against 64 KiB of capacity in the 512 cycles the
// MMA needs -- the kernel is tensor-bound.
//
// Pair tile: 256 weight rows x 256 batch rows.  CTA `rank` of the pair holds weight rows
// [n0 + 128*rank, +128) (its 128 TMEM lanes: A stages and the 256-column fp32 accumulator) and loads
// batch rows [m0 + 128*rank, +128) of X (its half of the B operand).
//
// Roles per CTA (320 threads):
//   warp 0      TMA producer: this CTA's half of the X tile [128 x 64], SWIZZLE_128B
//   warp 1      pair leader (rank 0): issues tcgen05.mma.cta_group::2 [d], [a_tmem], b_desc and commits
//               stage-free / accumulator-ready mbarriers in both CTAs; in the other CTA the same warp
//               forwards "my X half and my A stage are in place" with a remote mbarrier arrive
//   warps 2..5  epilogue: tcgen05.ld of D^T (lane = weight row; the load of the next 32 columns overlaps the
//               conversion of the previous 32), fp16, transposed through one shared [256][128] staging tile,
//               256-byte row segments of Y written with 16-byte stores (and the same to peers in gather
//               mode).  Tensor memory is handed back to the MMA warp as soon as it has been read, before the
//               write-out.  Variants: GATED (SiLU(gate) * up over neighbouring lanes, [256][64] tile) and
//               row-parallel mode (the tile goes to the owner of its columns with one TMA tensor store).
//   warps 6..9  dequant: thread (quarter, lane) owns weight row 32*quarter + lane
//
// Schedule: the K loops of all tiles are cut into units and dealt out evenly over the CTA pairs; a pair's
// two partial pieces are computed first, go to the workspace as fp32 and are summed in pair order by the
// contributor that arrives last (see take_segment and the epilogue).  Without a workspace: whole tiles.
//
// TMEM columns: [0, 256) accumulator, [256 + 64*s, +64) A stage s (two 64-wide K sub-steps).  No TMA load uses
// cluster multicast.  Every mbarrier wait is bounded (see tensor2.cu).
#include "tc_ptx.cuh"

namespace vqg {

using namespace tc;

namespace {

constexpr int BMH = 128;         // batch rows of X loaded per CTA (half of the pair's 256)
constexpr int BM = 256;          // batch rows per pair tile (MMA N dimension)
constexpr int BNH = 128;         // weight rows per CTA (its TMEM lanes)
constexpr int BN = 256;          // weight rows per pair tile (MMA M dimension)
constexpr int BK = 64;
constexpr int kThreads = 320;
constexpr int kDequantWarp0 = 6;
constexpr int kDequantThreads = 128;
constexpr uint32_t kXBytes = BMH * BK * 2;          // 16 KiB
constexpr uint32_t kImageBytes = 32 * 1024;
constexpr uint32_t kStagingBytes = 256 * 256;       // [256 batch rows][128 weight rows] fp16, shared by the 4 epilogue warps
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCols = 256;                  // accumulator columns; A stages follow
constexpr uint32_t kAColsPerStage = BK / 2;         // 32 columns: two fp16 per 32-bit column

struct TsParams {
  const unsigned char* idx;  // [N, K/v] uint8
  const __half* cb;          // [G, C, v]
  const unsigned char* idx2; // residual weights: indices and codebooks of the second stage (RESID kernels)
  const __half* cb2;
  __half* y;
  int* status;
  int M, N, K, C;
  int rows_per_cb;
  long long ld_y;
  int m_tiles, n_tiles;      // in 256 x 256 pair tiles
  // Schedule: the K loop of every tile is cut into `units_per_tile` units of `unit_stages` pipeline stages;
  // the tiles*units_per_tile units are dealt out evenly and contiguously, pair b taking
  // [b*q + min(b, r), +q + (b < r)).  units_per_tile == 1 keeps whole tiles per pair (no workspace needed).
  int unit_stages, units_per_tile, q, r;
  float* ws_partial;         // [pair][first/last segment][rank][256 batch rows][128 weight rows] fp32
  int* ws_counter;           // [tile][rank] arrivals of contributors; zero between calls
  int n_peers;
  __half* peer_y[8];
  __half* mc_y;              // multicast address of the output block (gather through the switch), or null
  // row-parallel mode: the tile goes, as this rank's partial sum, to the buffer of the rank that owns its
  // columns (tensor map `owner` of PeerMaps, local or peer memory) and nowhere else
  int n_owners, owner_cols;
};

__device__ __forceinline__ int pair_begin(int b, int q, int r) { return b * q + (b < r ? b : r); }
// pair that owns unit u
__device__ __forceinline__ int pair_of_unit(int u, int q, int r) {
  const int big = r * (q + 1);
  return u < big ? u / (q + 1) : r + (u - big) / q;
}

// Tensor maps of the owners' partial-sum buffers (row-parallel mode): a finished tile goes to its owner with
// one TMA tensor store (no multicast; an ordinary asynchronous bulk store whose destination may be peer memory).
struct alignas(64) PeerMaps {
  CUtensorMap m[8];
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(c0), "r"(c1), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// shared memory of all committed stores has been read (it may be rewritten)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all committed stores are complete
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// One contiguous piece of a pair's range inside one tile.
struct Segment {
  int tile, kt_begin, kt_end;   // pipeline stages [kt_begin, kt_end) of the tile's K loop
  bool whole;                   // the piece is the whole tile
  int start;                    // first unit of the piece
};
// Takes the next piece off the remaining range [lo, hi).  A range that ends inside a tile gives up that
// last piece first (`from_back`, once), then is walked from the front: both pieces of a tile shared by
// pairs b and b+1 are then computed at the start of the kernel, the sum of their partials overlaps the
// main loop of whoever arrives second, and every pair ends on a whole tile at the same time.
__device__ __forceinline__ Segment take_segment(int& lo, int& hi, bool& from_back, const TsParams& p) {
  Segment g;
  int end;
  const bool rev = from_back;
  from_back = false;
  if (!rev) {
    g.tile = lo / p.units_per_tile;
    const int t0 = g.tile * p.units_per_tile;
    g.start = lo;
    end = min(hi, t0 + p.units_per_tile);
    lo = end;
  } else {
    g.tile = (hi - 1) / p.units_per_tile;
    const int t0 = g.tile * p.units_per_tile;
    g.start = max(lo, t0);
    end = hi;
    hi = g.start;
  }
  const int t0 = g.tile * p.units_per_tile;
  g.kt_begin = (g.start - t0) * p.unit_stages;
  g.kt_end = (end - t0) * p.unit_stages;
  g.whole = (g.start == t0) && (end == t0 + p.units_per_tile);
  return g;
}

// The pieces of a pair's range in the order they are worked on; every role of the kernel walks them the same way.
// Both partial pieces come first, then the whole tiles.  Even pairs take the piece at the END of their range
// first, odd pairs the piece at the START: the tile shared by an even pair b and the odd pair b+1 then gets both of
// its pieces at the very start of the kernel and is complete after max(l, 1 - l) of a tile time (l = the even pair's
// share of it) instead of after both pairs have done both of their pieces -- in gather mode the first output crosses
// the link that much earlier.  (The other half of the shared tiles is complete when the pieces are, as before.)
struct Walk {
  int lo, hi;
  bool back_pending, front_first;
  __device__ __forceinline__ Walk(int pair_id, const TsParams& p) {
    lo = pair_begin(pair_id, p.q, p.r);
    hi = pair_begin(pair_id + 1, p.q, p.r);
    back_pending = (hi % p.units_per_tile) != 0;
    front_first = (pair_id & 1) != 0 && (lo % p.units_per_tile) != 0;
  }
  __device__ __forceinline__ bool next(Segment& g, const TsParams& p) {
    if (lo >= hi) return false;
    bool rev = false;
    if (front_first) front_first = false;           // the piece at the start of the range
    else if (back_pending) { rev = true; back_pending = false; }
    g = take_segment(lo, hi, rev, p);
    return true;
  }
};

// kind::f16, A = B = fp16, D = fp32, both K-major, M = 256 weight rows (pair), N = 256 batch rows
constexpr uint32_t kIdescTs = (1u << 4) | (static_cast<uint32_t>(BM >> 3) << 17) | (static_cast<uint32_t>(BN >> 4) << 24);

template <int STAGES, int KS, int IMAGES = 1>
struct TsSmem {
  static constexpr uint32_t kImage = STAGES * KS * kXBytes;
  static constexpr uint32_t kStaging = kImage + IMAGES * kImageBytes;
  static constexpr uint32_t kBars = kStaging + kStagingBytes;
  // full[S], empty[S], acc_full, acc_empty, dequant rendezvous, epilogue rendezvous
  static constexpr uint32_t kTmemSlot = kBars + (2 * STAGES + 4) * 8;
  static constexpr uint32_t kTotal = kTmemSlot + 16;
};

__device__ __forceinline__ void tc_mma_f16_pair_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 registers -> 32 consecutive tensor-memory columns of this thread's lane
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

// KS: 64-wide K sub-tiles per pipeline stage (a stage is KS*64 K values: fewer barrier round trips and
// commits per MMA for the single issuing thread).
// fp32 SiLU(g) * u of one (gate, up) pair of accumulators
__device__ __forceinline__ float swiglu(float g, float u) { return g / (1.0f + __expf(-g)) * u; }

// fp16 addition of two packed pairs, round to nearest even, subnormals kept: the rule of the residual format
__device__ __forceinline__ uint32_t hadd2_bits(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// GATED: weight rows come in (gate, up) pairs -- row 2i is gate row i, row 2i+1 is up row i -- and the
// epilogue writes SiLU(X g_i) * (X u_i) into output column i, so Y is [M, N/2] and the two products of a
// gated MLP's first half never reach memory.
// RESID: residual (two-codebook) weights, W = fp16(cb0[idx0] + cb1[idx1]): a dequant thread looks both entries
// up (two resident images, two index streams) and adds them with HADD2 before the tcgen05.st, so the tensor
// core sees ordinary fp16 weights.  One X stage less than the plain kernel makes room for the second image.
template <int V, int STAGES, int KS, bool GATED = false, bool RESID = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
vq_tensor_ts_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ PeerMaps peer_maps,
                    const TsParams p) {
  using L = TsSmem<STAGES, KS, RESID ? 2 : 1>;
  constexpr uint32_t kStageCols = KS * kAColsPerStage;
  constexpr uint32_t kStageXBytes = KS * kXBytes;
  static_assert(kAccCols + STAGES * kStageCols <= kTmemCols, "A stages do not fit tensor memory");
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;   // SWIZZLE_128B tiles need 1024-byte alignment
  unsigned char* base_ptr = smem_dyn + (base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();         // 0 = pair leader
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  auto x_addr = [&](int s) { return base + s * kStageXBytes; };
  // full[s]: this CTA's X half has landed (TMA, 1 arrival + bytes) and its 4 dequant warps have written
  // their A columns; in the leader one more arrival says the same of the second CTA.  One wait per stage.
  auto bar_full = [&](int s) { return base + L::kBars + 8 * s; };
  auto bar_empty = [&](int s) { return base + L::kBars + 8 * (STAGES + s); };
  const uint32_t bar_acc_full = base + L::kBars + 8 * (2 * STAGES);
  const uint32_t bar_acc_empty = base + L::kBars + 8 * (2 * STAGES + 1);
  const uint32_t bar_dq = base + L::kBars + 8 * (2 * STAGES + 2);
  const uint32_t bar_epi = base + L::kBars + 8 * (2 * STAGES + 3);
  // shared::cluster address of the same offset in the other CTA = local address + a constant
  const uint32_t to_peer = map_to_cta(base, rank ^ 1u) - base;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::kTmemSlot);

  // a kernel launched behind this one with programmatic stream serialisation (the cross-GPU barrier that ends a
  // sharded step) may take its place on an SM now; it waits for this grid to complete before it does anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1 + kDequantThreads / 32 + (rank == 0 ? 1 : 0));
      mbar_init(bar_empty(s), 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 8);   // 4 epilogue warps in each CTA of the pair
    mbar_init(bar_dq, kDequantThreads);
    mbar_init(bar_epi, 4);
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
      Walk walk(pair_id, p);
      Segment g;
      while (ok && walk.next(g, p)) {
        const int m0 = (g.tile % p.m_tiles) * BM + static_cast<int>(rank) * BMH;
        for (int kt = g.kt_begin; kt < g.kt_end; ++kt) {
          if (!(ok = mbar_wait_cluster(bar_empty(stage), phase ^ 1, p.status, DS_STAGE_EMPTY_TIMEOUT))) break;
          mbar_expect_tx(bar_full(stage), kStageXBytes);
#pragma unroll
          for (int u = 0; u < KS; ++u)
            tma_load_2d(x_addr(stage) + u * kXBytes, &tmap_x, (kt * KS + u) * BK, m0, bar_full(stage));
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
        uint32_t acc_phase = 0;
        Walk walk(pair_id, p);
        Segment g;
        while (ok && walk.next(g, p)) {
          if (!(ok = mbar_wait_cluster(bar_acc_empty, acc_phase ^ 1, p.status, DS_ACC_EMPTY_TIMEOUT))) break;
          tc_fence_after();
          for (int kt = g.kt_begin; kt < g.kt_end; ++kt) {
            if (!(ok = mbar_wait_cluster(bar_full(stage), phase, p.status, DS_TMA_FULL_TIMEOUT))) break;
            tc_fence_after();
            const uint32_t a_t = tmem_base + kAccCols + static_cast<uint32_t>(stage) * kStageCols;
#pragma unroll
            for (int u = 0; u < KS; ++u) {
              const uint64_t bd = make_desc(x_addr(stage) + u * kXBytes);
#pragma unroll
              for (int k = 0; k < BK / 16; ++k)   // 16 K values = 8 columns of A, 32 bytes of the X rows
                tc_mma_f16_pair_ts(tmem_base, a_t + u * kAColsPerStage + 8 * k, bd + 2 * k, kIdescTs,
                                   ((kt - g.kt_begin) | u | k) != 0 ? 1u : 0u);
            }
            // the stage (X tile and A columns) is free in both CTAs once these MMAs have read it
            tc_commit_pair(bar_empty(stage));
            tc_commit_pair(bar_empty(stage) + to_peer);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          tc_commit_pair(bar_acc_full);
          tc_commit_pair(bar_acc_full + to_peer);
          acc_phase ^= 1;
        }
      } else {
        // ------------------------------- forwarder (second CTA) -----------------------------
        Walk walk(pair_id, p);
        Segment g;
        while (ok && walk.next(g, p)) {
          for (int kt = g.kt_begin; kt < g.kt_end; ++kt) {
            if (!(ok = mbar_wait(bar_full(stage), phase, p.status, DS_TMA_FULL_TIMEOUT))) break;
            mbar_arrive_remote(bar_full(stage) + to_peer);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp < kDequantWarp0) {
    // ------------------------------- epilogue -----------------------------------------------
    // D^T: lane = weight row, column = batch row.  The four warps transpose the CTA's 128 weight rows
    // through one [256][128] fp16 tile and write Y in 256-byte row segments (whole lines, also on NVLink).
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t acc_phase = 0, epi_phase = 0;
    bool ok = true;
    const uint32_t leader_acc_empty = bar_acc_empty + (rank == 0 ? 0u : to_peer);
    unsigned char* stg = base_ptr + L::kStaging;
    auto epi_sync = [&]() -> bool {   // bounded rendezvous of the four epilogue warps
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_epi);
      const bool done = mbar_wait(bar_epi, epi_phase, p.status, DS_EPILOGUE_SYNC_TIMEOUT);
      epi_phase ^= 1;
      return done;
    };
    volatile int* last_flag = reinterpret_cast<volatile int*>(base_ptr + L::kTmemSlot + 8);
    constexpr int OUT_COLS = GATED ? BNH / 2 : BNH;      // output columns of this CTA's half tile
    constexpr int ROW_BYTES = OUT_COLS * 2;              // one staged row of the tile
    constexpr size_t kPartialFloats = static_cast<size_t>(BM) * BNH;   // one CTA's share of a pair tile
    Walk walk(pair_id, p);
    Segment g;
    while (ok && walk.next(g, p)) {
      const int tile = g.tile;
      const int m0 = (tile % p.m_tiles) * BM;
      const int n0 = ((tile / p.m_tiles) * BN + static_cast<int>(rank) * BNH) / (GATED ? 2 : 1);   // first output column
      const int n_out = GATED ? p.N / 2 : p.N;
      if (!(ok = mbar_wait_cluster(bar_acc_full, acc_phase, p.status, DS_ACC_FULL_TIMEOUT))) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      bool released = false;
      if (g.whole) {
        // two register buffers: the tensor-memory load of the next 32 columns runs while these are converted
        // and stored, and tensor memory is handed back as soon as the last load has landed
        uint32_t ra[32], rb[32];
        auto put = [&](int c, const uint32_t (&r)[32]) {
          if constexpr (GATED) {
            // lanes 2i / 2i+1 hold gate / up row i: the even lane takes its neighbour's value and writes column i
            __half* col = reinterpret_cast<__half*>(stg) + (c * 32) * OUT_COLS + ((quarter * 32 + lane) >> 1);
            // one exchange per two batch columns: the even lane finishes column j, the odd lane column j + 1
            const bool odd = (lane & 1) != 0;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float send = odd ? __uint_as_float(r[j]) : __uint_as_float(r[j + 1]);
              const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
              const float y = odd ? swiglu(recv, __uint_as_float(r[j + 1])) : swiglu(__uint_as_float(r[j]), recv);
              col[(j + (odd ? 1 : 0)) * OUT_COLS] = __float2half_rn(y);
            }
          } else {
            __half* col = reinterpret_cast<__half*>(stg) + (c * 32) * 128 + quarter * 32 + lane;   // T[m][weight row]
#pragma unroll
            for (int j = 0; j < 32; ++j) col[j * 128] = __float2half_rn(__uint_as_float(r[j]));
          }
        };
        if constexpr (!GATED) {
          // The whole row is converted to fp16 in registers first (two batch columns per register) and tensor
          // memory handed back before a single shared-memory store is issued: the stores queue behind the dequant
          // warps' lookups, and every cycle they take before the release is a cycle the tensor pipe stands still.
          uint32_t hp[BM / 2];
          uint32_t qa[16], qb[16];                 // 16 columns per load: the row itself takes 128 registers
          tmem_ld16_async(t_row, qa);
#pragma unroll
          for (int c = 0; c < BM / 16; c += 2) {
            tmem_ld_wait16(qa);
            tmem_ld16_async(t_row + (c + 1) * 16, qb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const __half2 h = __floats2half2_rn(__uint_as_float(qa[2 * j]), __uint_as_float(qa[2 * j + 1]));
              hp[c * 8 + j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            tmem_ld_wait16(qb);
            if (c + 2 < BM / 16) {
              tmem_ld16_async(t_row + (c + 2) * 16, qa);
            } else {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_remote(leader_acc_empty);
              released = true;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const __half2 h = __floats2half2_rn(__uint_as_float(qb[2 * j]), __uint_as_float(qb[2 * j + 1]));
              hp[(c + 1) * 8 + j] = *reinterpret_cast<const uint32_t*>(&h);
            }
          }
          unsigned short* col = reinterpret_cast<unsigned short*>(stg) + quarter * 32 + lane;   // T[m][weight row]
#pragma unroll
          for (int q = 0; q < BM / 2; ++q) {
            col[(2 * q) * 128] = static_cast<unsigned short>(hp[q] & 0xffffu);
            col[(2 * q + 1) * 128] = static_cast<unsigned short>(hp[q] >> 16);
          }
        } else {
        tmem_ld32_async(t_row, ra);
#pragma unroll 1
        for (int c = 0; c < BM / 32; c += 2) {
          tmem_ld_wait(ra);
          tmem_ld32_async(t_row + (c + 1) * 32, rb);
          put(c, ra);
          tmem_ld_wait(rb);
          if (c + 2 < BM / 32) {
            tmem_ld32_async(t_row + (c + 2) * 32, ra);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(leader_acc_empty);
            released = true;
          }
          put(c + 1, rb);
        }
        }
      } else {
        // a piece of a tile: the fp32 partial goes to this pair's slot (0 when the pair's range begins
        // inside the tile, 1 when it begins at or before the tile's first unit)
        const int slot = (g.start > tile * p.units_per_tile) ? 0 : 1;
        float* part = p.ws_partial + ((static_cast<size_t>(pair_id) * 2 + slot) * 2 + rank) * kPartialFloats + quarter * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BM / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(part + static_cast<size_t>(c * 32 + j) * BNH, __uint_as_float(r[j]));
        }
      }
      // tensor memory has been read: the next tile's MMAs may overwrite it while Y is written out
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(leader_acc_empty);
      }
      acc_phase ^= 1;
      if (!g.whole) {
        // The contributor that arrives last sums the partials of all contributors (consecutive pairs) in
        // pair order, so the result does not depend on who that is.
        const int t0u = tile * p.units_per_tile;
        const int b_first = pair_of_unit(t0u, p.q, p.r);
        const int b_last = pair_of_unit(t0u + p.units_per_tile - 1, p.q, p.r);
        __threadfence();
        if (!(ok = epi_sync())) break;   // all four warps' partials are written and fenced
        if (warp == 2 && lane == 0) {
          int* ctr = p.ws_counter + tile * 2 + static_cast<int>(rank);
          const int old = atomicAdd(ctr, 1);
          const int last = (old == b_last - b_first);
          if (last) *ctr = 0;            // leave the counter zero for the next call
          *last_flag = last;
        }
        if (!(ok = epi_sync())) break;
        const int last = *last_flag;
        if (!last) {
          if (!(ok = epi_sync())) break; // the flag is rewritten only after everyone has read it
          continue;
        }
        __threadfence();
        {
          // thread -> four consecutive weight rows of one batch row; 16 independent 16-byte loads in flight
          // per thread and contributor (a dependent chain of L2 round trips would dominate otherwise)
          const int et = quarter * 32 + lane;          // 0..127
          const int row4 = (et & 31) * 4, msub = et >> 5;
          constexpr int INFL = 16;
#pragma unroll 1
          for (int i0 = 0; i0 < BM / 4; i0 += INFL) {
            float4 sum[INFL];
#pragma unroll
            for (int j = 0; j < INFL; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int b = b_first; b <= b_last; ++b) {
              const int slot = (pair_begin(b, p.q, p.r) > t0u) ? 0 : 1;
              const float* src = p.ws_partial + ((static_cast<size_t>(b) * 2 + slot) * 2 + rank) * kPartialFloats + row4;
              float4 v[INFL];
#pragma unroll
              for (int j = 0; j < INFL; ++j)
                v[j] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(4 * (i0 + j) + msub) * BNH));
#pragma unroll
              for (int j = 0; j < INFL; ++j) {
                sum[j].x += v[j].x; sum[j].y += v[j].y; sum[j].z += v[j].z; sum[j].w += v[j].w;
              }
            }
#pragma unroll
            for (int j = 0; j < INFL; ++j) {
              if constexpr (GATED) {   // the thread's four weight rows are two (gate, up) pairs
                const __half2 o2 = __floats2half2_rn(swiglu(sum[j].x, sum[j].y), swiglu(sum[j].z, sum[j].w));
                *reinterpret_cast<uint32_t*>(stg + (4 * (i0 + j) + msub) * ROW_BYTES + row4) = *reinterpret_cast<const uint32_t*>(&o2);
              } else {
                const __half2 lo2 = __floats2half2_rn(sum[j].x, sum[j].y), hi2 = __floats2half2_rn(sum[j].z, sum[j].w);
                uint2 o;
                o.x = *reinterpret_cast<const uint32_t*>(&lo2);
                o.y = *reinterpret_cast<const uint32_t*>(&hi2);
                *reinterpret_cast<uint2*>(stg + (4 * (i0 + j) + msub) * 256 + row4 * 2) = o;
              }
            }
          }
        }
      }
      const bool tma_out = p.n_owners > 0;
      if (tma_out) fence_async_smem();   // this thread's staging writes become visible to the TMA unit
      if (!(ok = epi_sync())) break;   // the whole tile is in shared memory
      if (tma_out && warp == 2 && lane == 0) {
        // row-parallel: this rank's partial tile goes to the owner of these output columns with one tensor
        // store (rows beyond M are clipped by the tensor map)
        const int o = n0 / p.owner_cols;
        tma_store_2d(&peer_maps.m[o], n0 - o * p.owner_cols, m0, smem_u32(stg));
        tma_store_commit();
      }
      if (p.n_owners == 0) {
        constexpr int LPR = ROW_BYTES / 16, RPW = 32 / LPR;   // lanes per staged row, rows per warp instruction
        const int rsel = lane / LPR, chunk = lane % LPR;
        const int ncol = n0 + chunk * 8;
#pragma unroll 4
        for (int i = 0; i < BM / (4 * RPW); ++i) {
          const int m = (4 * i + quarter) * RPW + rsel;
          if (m0 + m < p.M && ncol < n_out) {
            const uint4 v = *reinterpret_cast<const uint4*>(stg + m * ROW_BYTES + chunk * 16);
            const size_t off = static_cast<size_t>(m0 + m) * p.ld_y + ncol;
            if (p.mc_y) {
              // gather through the switch: ONE 16-byte multimem store to the multicast mapping of the ranks'
              // Y buffers; NVSwitch writes it into every rank's copy (this rank's too), so the SM issues one
              // store per 16 bytes instead of one per rank and the link carries the block out once
              asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.mc_y + off),
                           "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                           "f"(__uint_as_float(v.w)) : "memory");
              continue;
            }
            *reinterpret_cast<uint4*>(p.y + off) = v;
            // gather mode: the same 16 bytes to every peer's copy of Y.  (One TMA tensor store per peer from
            // the staging tile was measured slower: 265 against 219 us per step on 8 GPUs, 223 against 217 on
            // 4 -- the queued 64 KiB stores hold up the TMA loads of X.)
            for (int q = 0; q < p.n_peers; ++q) *reinterpret_cast<uint4*>(p.peer_y[q] + off) = v;
          }
        }
      }
      if (tma_out && warp == 2 && lane == 0) tma_store_wait_read();   // the TMA unit has read the tile
      if (!(ok = epi_sync())) break;   // the tile is rewritten by the next tile's transposition
    }
    if (p.n_owners > 0 && warp == 2 && lane == 0) tma_store_wait_all();   // stores done before the kernel ends
  } else {
    // ------------------------------- dequant warps ------------------------------------------
    constexpr int ENTRY_LOG2 = (V == 4) ? 3 : 4;       // bytes per codebook entry
    constexpr int REPS = 128 >> ENTRY_LOG2;             // replicas filling a 128-byte line
    constexpr int WPS = (BK / V) / 4;                   // index words per K step (uint8 indices)
    constexpr int GSTEPS = 16 / WPS;                    // K steps per 64-byte granule
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                  // weight row inside the CTA = TMEM lane
    const int tix = threadIdx.x - kDequantWarp0 * 32;   // 0..127, for cooperative copies
    const int J = p.K / V;                              // index bytes per weight row
    unsigned char* image = base_ptr + L::kImage;
    const uint32_t img = base + L::kImage + ((lane & (REPS - 1)) << ENTRY_LOG2);
    const uint32_t a_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kAccCols;

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
    Walk walk(pair_id, p);
    Segment g;
    while (ok && walk.next(g, p)) {
      const int n_half0 = (g.tile / p.m_tiles) * BN + static_cast<int>(rank) * BNH;
      const int n = n_half0 + r;
      const bool row_valid = n < p.N;
      const int group = (n_half0 < p.N ? n_half0 : p.N - 1) / p.rows_per_cb;
      if (group != cur_group) {
        cur_group = group;
        if (!(ok = dq_sync())) break;   // every thread has finished its lookups in the old image
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.cb) + (static_cast<size_t>(group) * p.C << ENTRY_LOG2);
        if (V == 4) {
          for (int u = tix; u < p.C * (REPS / 2); u += kDequantThreads) {
            const uint2 e = __ldg(reinterpret_cast<const uint2*>(src) + u / (REPS / 2));
            reinterpret_cast<uint4*>(image)[u] = make_uint4(e.x, e.y, e.x, e.y);
          }
        } else {
          for (int u = tix; u < p.C * REPS; u += kDequantThreads)
            reinterpret_cast<uint4*>(image)[u] = __ldg(reinterpret_cast<const uint4*>(src) + u / REPS);
        }
        if constexpr (RESID) {   // the second stage's codebook of the same group, behind the first image
          const unsigned char* src2 = reinterpret_cast<const unsigned char*>(p.cb2) + (static_cast<size_t>(group) * p.C << ENTRY_LOG2);
          unsigned char* image2 = image + kImageBytes;
          if (V == 4) {
            for (int u = tix; u < p.C * (REPS / 2); u += kDequantThreads) {
              const uint2 e = __ldg(reinterpret_cast<const uint2*>(src2) + u / (REPS / 2));
              reinterpret_cast<uint4*>(image2)[u] = make_uint4(e.x, e.y, e.x, e.y);
            }
          } else {
            for (int u = tix; u < p.C * REPS; u += kDequantThreads)
              reinterpret_cast<uint4*>(image2)[u] = __ldg(reinterpret_cast<const uint4*>(src2) + u / REPS);
          }
        }
        if (!(ok = dq_sync())) break;
      }

      const unsigned char* row_ptr = p.idx + static_cast<size_t>(row_valid ? n : 0) * J;
      uint32_t cur[16], nxt[16];
      // second index stream of the residual format (one 16-register buffer: its loads are issued a granule
      // ahead like the first stream's, straight into the buffer the next granule reads)
      constexpr int R2 = RESID ? 16 : 1;
      uint32_t cur2[R2], nxt2[R2];
      auto load_granule_from = [&](const unsigned char* rp, int gi, uint32_t* dst) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 t = make_uint4(0, 0, 0, 0);
          const int byte0 = gi * 64 + q * 16;
          if (row_valid && byte0 + 16 <= J) t = __ldg(reinterpret_cast<const uint4*>(rp + byte0));
          dst[4 * q] = t.x; dst[4 * q + 1] = t.y; dst[4 * q + 2] = t.z; dst[4 * q + 3] = t.w;
        }
      };
      const unsigned char* row_ptr2 = RESID ? p.idx2 + static_cast<size_t>(row_valid ? n : 0) * J : nullptr;
      auto load_granule = [&](int gi, uint32_t (&dst)[16]) {
        load_granule_from(row_ptr, gi, dst);
        if constexpr (RESID) load_granule_from(row_ptr2, gi, nxt2);
      };
      // a unit is a whole number of 64-byte index granules unless it is the whole tile
      const int ks_begin = g.kt_begin * KS, ks_end = g.kt_end * KS;    // 64-wide sub-steps of the piece
      const int gi_begin = ks_begin / GSTEPS, ngran = (ks_end + GSTEPS - 1) / GSTEPS;
      load_granule(gi_begin, nxt);
      for (int gi = gi_begin; ok && gi < ngran; ++gi) {
#pragma unroll
        for (int i = 0; i < 16; ++i) cur[i] = nxt[i];
        if constexpr (RESID) {
#pragma unroll
          for (int i = 0; i < 16; ++i) cur2[i] = nxt2[i];
        }
        if (gi + 1 < ngran) load_granule(gi + 1, nxt);
#pragma unroll
        for (int st = 0; st < GSTEPS; ++st) {
          const int ks = gi * GSTEPS + st;                 // 64-wide sub-step; KS of them make a stage
          if (ks >= ks_end) break;
          // 64 K values of this row: 32 registers, in K order = 32 columns of the A stage
          uint32_t a[32];
          if (V == 4) {
#pragma unroll
            for (int w = 0; w < WPS; ++w) {
              const uint32_t word = cur[st * WPS + w];
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const uint32_t c0 = (word >> (8 * b)) & 0xffu;
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(a[8 * w + 2 * b]), "=r"(a[8 * w + 2 * b + 1]) : "r"(img + (c0 << 7)));
                if constexpr (RESID) {
                  const uint32_t c1 = (cur2[st * WPS + w] >> (8 * b)) & 0xffu;
                  uint32_t e0, e1;
                  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(e0), "=r"(e1) : "r"(img + kImageBytes + (c1 << 7)));
                  a[8 * w + 2 * b] = hadd2_bits(a[8 * w + 2 * b], e0);
                  a[8 * w + 2 * b + 1] = hadd2_bits(a[8 * w + 2 * b + 1], e1);
                }
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
                             : "=r"(a[16 * w + 4 * b]), "=r"(a[16 * w + 4 * b + 1]), "=r"(a[16 * w + 4 * b + 2]), "=r"(a[16 * w + 4 * b + 3])
                             : "r"(img + (c0 << 7)));
                if constexpr (RESID) {
                  const uint32_t c1 = (cur2[st * WPS + w] >> (8 * b)) & 0xffu;
                  uint32_t e0, e1, e2, e3;
                  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(e0), "=r"(e1), "=r"(e2), "=r"(e3)
                               : "r"(img + kImageBytes + (c1 << 7)));
                  a[16 * w + 4 * b] = hadd2_bits(a[16 * w + 4 * b], e0);
                  a[16 * w + 4 * b + 1] = hadd2_bits(a[16 * w + 4 * b + 1], e1);
                  a[16 * w + 4 * b + 2] = hadd2_bits(a[16 * w + 4 * b + 2], e2);
                  a[16 * w + 4 * b + 3] = hadd2_bits(a[16 * w + 4 * b + 3], e3);
                }
              }
            }
          }
          // (the lookups above overlap the wait for the stage)
          const int sub = st % KS;                          // GSTEPS is a multiple of KS
          if (sub == 0) {
            if (!(ok = mbar_wait_cluster(bar_empty(stage), phase ^ 1, p.status, DS_STAGE_EMPTY_TIMEOUT))) break;
            tc_fence_after();
          }
          tmem_st32(a_lane + static_cast<uint32_t>(stage) * kStageCols + sub * kAColsPerStage, a);
          if (sub == KS - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full(stage));
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  }

  // ------------------------------- teardown --------------------------------------------------
  // Nobody leaves before both CTAs are done: the leader's MMAs read the peer's shared and tensor memory
  // and both CTAs signal each other's mbarriers.
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

// fp16 row-major Y block [rows, cols] with leading dimension ld, box = the epilogue's staging tile
// [256 rows x 128 cols], no swizzle (the tile is dense in shared memory).
bool make_y_map(CUtensorMap* map, const void* ptr, int rows, int cols, long long ld) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {128, 256};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool tensor_ts_supported(const Problem& p) {
  if (p.M < 1 || p.N < 1 || p.K < 2 * BK || p.K % (2 * BK) != 0) return false;   // stages of 128 K values
  if (reinterpret_cast<uintptr_t>(p.x) % 16 || reinterpret_cast<uintptr_t>(p.y) % 16) return false;
  if (p.N % 32 != 0 || p.ld_y % 8 != 0) return false;
  if (!(p.v == 4 || p.v == 8) || p.idx_bytes != 1 || p.C < 1 || p.C > 256) return false;
  if ((p.K / p.v) % 16 != 0) return false;  // 16-byte index loads per row
  if (reinterpret_cast<uintptr_t>(p.idx) % 16 || reinterpret_cast<uintptr_t>(p.cb) % 16) return false;
  const bool single = p.rows_per_cb >= p.N;
  if (!single && p.rows_per_cb % 128 != 0) return false;
  return true;
}

namespace {
int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 1 ? sms : 148;
}
constexpr size_t kPairPartialBytes = 2 /*slots*/ * 2 /*ranks*/ * static_cast<size_t>(BM) * BNH * sizeof(float);
// pipeline stages per schedule unit: a whole number of the dequant threads' 64-byte index granules
int unit_stages_for(int v) { return v == 4 ? 2 : 4; }
}  // namespace

// Counters plus two fp32 partial tiles per CTA pair: with it the K loops are dealt out evenly over the
// pairs (no partly filled last wave); without it every tile is computed by one pair.
size_t tensor_ts_workspace_bytes(const Problem& p) {
  if (!tensor_ts_supported(p)) return 0;
  return kCounterBytes + static_cast<size_t>(sm_count() / 2) * kPairPartialBytes;
}

int launch_tensor_ts(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s, bool gated) {
  if (!tensor_ts_supported(p)) return VQG_ERR_UNSUPPORTED;
  if (gated && (p.n_peers != 0 || p.N % 2 != 0)) return VQG_ERR_UNSUPPORTED;
  CUtensorMap mx;
  if (!make_map(&mx, p.x, p.M, p.K)) return VQG_ERR_LAUNCH;
  PeerMaps pm{};
  if (p.n_peers < 0 || p.n_peers > 7) return VQG_ERR_BAD_ARG;
  for (int q = 0; q < p.n_peers; ++q)
    if (reinterpret_cast<uintptr_t>(p.peer_y[q]) % 16) return VQG_ERR_BAD_ARG;
  if (p.n_owners > 0) {
    if (p.n_peers != 0 || gated || p.n_owners > 8 || p.owner_cols % 128 != 0 ||
        static_cast<long long>(p.n_owners) * p.owner_cols != p.N)
      return VQG_ERR_UNSUPPORTED;
    for (int o = 0; o < p.n_owners; ++o) {
      if (!p.owner_part[o] || reinterpret_cast<uintptr_t>(p.owner_part[o]) % 16) return VQG_ERR_BAD_ARG;
      if (!make_y_map(&pm.m[o], p.owner_part[o], p.M, p.owner_cols, p.owner_cols)) return VQG_ERR_LAUNCH;
    }
  }
  TsParams tp{};
  tp.idx = static_cast<const unsigned char*>(p.idx);
  tp.cb = p.cb;
  tp.y = p.y;
  tp.status = device_status_ptr();
  tp.M = p.M; tp.N = p.N; tp.K = p.K; tp.C = p.C;
  tp.rows_per_cb = p.rows_per_cb >= p.N ? p.N : p.rows_per_cb;
  tp.ld_y = p.ld_y;
  tp.m_tiles = (p.M + BM - 1) / BM;
  tp.n_tiles = (p.N + BN - 1) / BN;
  tp.n_peers = p.n_peers;
  for (int i = 0; i < 8; ++i) tp.peer_y[i] = p.peer_y[i];
  tp.mc_y = p.mc_y;
  tp.n_owners = p.n_owners;
  tp.owner_cols = p.owner_cols;
  const int max_pairs = sm_count() / 2;
  const int tiles = tp.m_tiles * tp.n_tiles;
  const int ksteps = p.K / (2 * BK);
  const int us = unit_stages_for(p.v);
  const bool split = ws && reinterpret_cast<uintptr_t>(ws) % 256 == 0 &&
                     ws_bytes >= kCounterBytes + static_cast<size_t>(max_pairs) * kPairPartialBytes &&
                     ksteps % us == 0 && ksteps / us > 1 && tiles % max_pairs != 0 &&
                     static_cast<size_t>(tiles) * 2 * sizeof(int) <= kCounterBytes;
  tp.unit_stages = split ? us : ksteps;
  tp.units_per_tile = split ? ksteps / us : 1;
  const long long units = static_cast<long long>(tiles) * tp.units_per_tile;
  if (units > 0x7fffffffLL) return VQG_ERR_UNSUPPORTED;
  const int pairs = units < max_pairs ? static_cast<int>(units) : max_pairs;
  tp.q = static_cast<int>(units / pairs);
  tp.r = static_cast<int>(units % pairs);
  tp.ws_counter = split ? static_cast<int*>(ws) : nullptr;
  tp.ws_partial = split ? reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + kCounterBytes) : nullptr;
  constexpr int S = 4, KS = 2;   // 4 stages of 128 K values: 128 KiB of X tiles, 4 x 64 TMEM columns of A
  constexpr int SR = 3;          // residual weights: 3 stages, the fourth's 32 KiB hold the second codebook image
  const bool resid = p.n_stages == 2;
  if (p.n_stages > 2 || (resid && gated)) return VQG_ERR_UNSUPPORTED;
  if (resid) {
    const int groups = (p.N + tp.rows_per_cb - 1) / tp.rows_per_cb;
    tp.idx2 = tp.idx + static_cast<size_t>(p.N) * (p.K / p.v);
    tp.cb2 = tp.cb + static_cast<size_t>(groups) * p.C * p.v;
  }
  const size_t smem = (resid ? TsSmem<SR, KS, 2>::kTotal : TsSmem<S, KS>::kTotal) + 1024;
  auto launch = [&](auto kernel) -> int {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return VQG_ERR_LAUNCH;
    kernel<<<2 * pairs, kThreads, smem, s>>>(mx, pm, tp);
    count_launch();
    return cuda_status(cudaGetLastError());
  };
  if (resid) return p.v == 4 ? launch(vq_tensor_ts_kernel<4, SR, KS, false, true>) : launch(vq_tensor_ts_kernel<8, SR, KS, false, true>);
  if (gated) return p.v == 4 ? launch(vq_tensor_ts_kernel<4, S, KS, true>) : launch(vq_tensor_ts_kernel<8, S, KS, true>);
  if (p.v == 4) return launch(vq_tensor_ts_kernel<4, S, KS>);
  return launch(vq_tensor_ts_kernel<8, S, KS>);
}

}  // namespace vqg
