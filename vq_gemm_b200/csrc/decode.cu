// Memory-bound VQ-GEMM for M <= 16 (decode / small batch), sm_100a.
//
// The problem is a GEMV-like stream over the index matrix: every index is read once from HBM
// and costs one shared-memory codebook lookup.  What this kernel is built around:
//
//   * index tiles arrive by TMA (cp.async.bulk.tensor.2d, no multicast) behind mbarriers, into a
//     PRIVATE ring of each warp: a warp owns one K slice (512 K values for M <= 4, 256 above) and
//     walks over the row blocks of its CTA, so its tiles are [8 or 16 rows] x [one slice] = 1 KiB,
//     several of them in flight, and no warp ever waits for another one while streaming.  The tile
//     is stored with the TMA swizzle that matches its row length (32/64/128 bytes), which makes the
//     16-byte reads of the eight rows of a unit conflict-free.  The first tiles are requested a few
//     hundred cycles into the kernel, before anything else is set up;
//   * the codebook of a row block's group sits in shared memory as a REPLICATED image: entry c,
//     replica r at byte  c*(R*2v) + r*2v , lane uses replica lane % R.  With R = 64/v
//     (C <= 256) a warp-wide lookup touches every bank exactly once per wavefront;
//   * looked-up entries go into mma.sync.m16n8k16 operand registers AS THEY ARRIVE -- no
//     conversion, shuffle or register move -- and accumulation is fp32 in the tensor core.  Thread
//     (g, t) of a warp owns weight row n0+g and a contiguous quarter of the warp's K slice.
//       form 1 (M <= 4)  16 bytes of codebook data (one v=8 entry, or two consecutive v=4 entries)
//         are the 4 registers of an A fragment: MMA row g sees K pairs {0-1, 4-5} of them, MMA row
//         g+8 sees pairs {2-3, 6-7}.  X is the B operand with two columns per batch row m:
//         column 2m carries X for the pairs of row g, column 2m+1 those of row g+8, so that
//         y[n0+g][m] = D[g][2m] + D[g+8][2m+1].  One MMA per 16 codebook bytes.  256 threads and at
//         most 128 registers: two launches fit an SM side by side, so with programmatic dependent
//         launch the whole prologue of launch i+1 (tiles in flight, image built) hides behind launch i;
//       forms 2/3 (M <= 8 / 16) a v=4 entry (or half a v=8 entry) is the 2-register B fragment of
//         column g; X (batch rows g and g+8) is the A operand.  One MMA per 8 codebook bytes.
//     The X fragments of a warp's slice are loaded once per K chunk, straight from global memory in
//     register order, and stay in registers;
//   * the partial tiles of a CTA's warps are summed in slice order through shared memory
//     (deterministic), one barrier per batch of row blocks; K > 4096 either walks the chunks with
//     running sums in shared memory (a CTA owns its rows for all of K) or, on matrices with few
//     row blocks, hands fp32 partials over through a workspace in which the last-arriving CTA of
//     a row block sums the chunks in chunk order (also deterministic).
//
// There is no reference counterpart: the reference requires M % 128 == 0
// (strategy_1/src.cu:221); the dequantisation rule is that of strategy_2/bsz128/src.cu:179-190.
#include <mutex>
#include <type_traits>

#include "tc_ptx.cuh"

namespace vqg {

namespace {

struct DecodeParams {
  const __half* x;
  const __half* cb;
  __half* y;
  float* ws_partial;   // [nchunks][M][N] fp32 (split-K through the workspace only)
  int* ws_counter;     // [row block groups]
  int* status;
  int M, N, K, C;
  long long ld_y;
  int nslices;         // K / KS
  int nchunks;         // K chunks a row block is summed over: kchunks * stages
  int kchunks;         // ceil(nslices / warps): chunks of K
  int ngroups;         // codebook groups of one stage
  int stage_rows;      // rows between the index matrices of consecutive residual stages (N)
  int rl;              // row lanes: super-units processed side by side by one CTA (warps / slices when K is short)
  int nrbg;            // items per chunk: ceil(N / (8 * SU * rl))
  int nslots;          // resident codebook images (1 or 2)
  int items_q, items_r; // items per CTA: q, and one more for the first r CTAs
  int ipg;             // items per codebook group
  int stages;          // tiles in flight per warp
  int batch;           // items per reduction batch (<= kMaxBatch)
  int bar_offset, img_offset, part_offset, acc_offset;   // byte offsets into the 1024-aligned shared memory
  unsigned inv_m, inv_rl;   // ceil(2^32 / M), ceil(2^32 / rl), 0 for a divisor of 1: t / M == umulhi(t, inv_m) for the small t in use
  int n_peers;
  __half* peer_y[8];
  // K > 4096 on matrices with many row blocks: a CTA owns a range of items for ALL K chunks (items_q/r then
  // partition the items of one chunk), walks the chunks one after the other and keeps the running sums of its
  // rows in shared memory at acc_offset -- no partial sums in global memory, no counters, no hand-over.
  int row_owned;
};

constexpr int kMaxBatch = 16;


// Geometry of one instantiation.
template <int V, int IB, int FORM>
struct Geo {
  static constexpr int NW = (FORM == 1) ? 8 : 16;      // warps per CTA
  static constexpr int NT = NW * 32;
  static constexpr int KS = (FORM == 1) ? 512 : 256;   // K values per warp slice
  static constexpr int TK = KS / 4;                    // K values per thread and unit (contiguous)
  static constexpr int SLABB = KS / V * IB;            // index bytes per row and slice: 128, 64 or 32
  static constexpr int TB = SLABB / 4;                 // index bytes per thread and row: 32, 16 or 8
  static constexpr int SU = (SLABB >= 128) ? 1 : 2;    // 8-row units per tile
  static constexpr int STAGE = 8 * SU * SLABB;         // tile bytes: 1024 (512 for 32-byte rows)
  static constexpr int XR = (FORM == 1) ? TK / 4 : (FORM == 2 ? TK / 2 : TK);   // X fragment registers per thread
  static constexpr int W64 = 64 / V * IB / 4;          // index words per 64 K values
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory loads by 32-bit address.  Not volatile, so the compiler may schedule them freely;
// `epoch` is a fake input that changes whenever the codebook image is rebuilt, which keeps a load
// from being moved across the barrier that publishes the new image.
__device__ __forceinline__ uint2 lds64(uint32_t addr, uint32_t epoch) {
  uint2 r;
  asm("ld.shared.v2.u32 {%0,%1}, [%2];  // %3" : "=r"(r.x), "=r"(r.y) : "r"(addr), "r"(epoch));
  return r;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr, uint32_t epoch) {
  uint4 r;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];  // %5" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr), "r"(epoch));
  return r;
}
// Index words out of a TMA tile: volatile, they must stay behind the wait on the tile's mbarrier.
__device__ __forceinline__ uint4 lds128_tile(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr) : "memory");
  return r;
}
__device__ __forceinline__ uint2 lds64_tile(uint32_t addr) {
  uint2 r;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr) : "memory");
  return r;
}

// 16-bit indices are held below `cmax` + 1 = C (a larger one -- malformed input -- would address past the image
// and end the launch); 8-bit ones cannot leave the 256-entry image region.
template <int IB>
__device__ __forceinline__ uint32_t idx_at(const uint32_t* w, int i, uint32_t cmax) {
  if constexpr (IB == 1) return __byte_perm(w[i >> 2], 0, 0x4440 + (i & 3));
  else return min(__byte_perm(w[i >> 1], 0, (i & 1) ? 0x4432 : 0x4410), cmax);
}

// The products of one thread for 64 of its K values and one 8-row unit: `w` holds the indices of those K values,
// `xf` the matching X fragment registers, `img` is the lane's replica inside the group's codebook image.
template <int V, int IB, int FORM, int ENTRY_SHIFT>
__device__ __forceinline__ void piece_mma(float (&acc)[4][4], const uint32_t* w, const uint32_t* xf,
                                          uint32_t img, uint32_t epoch, uint32_t cmax) {
  if constexpr (FORM == 1) {
    if constexpr (V == 4) {
      uint2 e[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = lds64(img + (idx_at<IB>(w, i, cmax) << ENTRY_SHIFT), epoch);
#pragma unroll
      for (int q = 0; q < 8; ++q)
        mma_16816(acc[q & 3], e[2 * q].x, e[2 * q].y, e[2 * q + 1].x, e[2 * q + 1].y, xf[2 * q], xf[2 * q + 1]);
    } else {
      uint4 e[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) e[i] = lds128(img + (idx_at<IB>(w, i, cmax) << ENTRY_SHIFT), epoch);
#pragma unroll
      for (int q = 0; q < 8; ++q) mma_16816(acc[q & 3], e[q].x, e[q].y, e[q].z, e[q].w, xf[2 * q], xf[2 * q + 1]);
    }
  } else {
    constexpr int XS = (FORM == 2) ? 2 : 4;
    if constexpr (V == 4) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {   // two halves of 8 lookups keep the register count down
        uint2 e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = lds64(img + (idx_at<IB>(w, 8 * hf + i, cmax) << ENTRY_SHIFT), epoch);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int ii = 8 * hf + i;
          if constexpr (FORM == 2) mma_16816(acc[i & 3], xf[XS * ii], 0u, xf[XS * ii + 1], 0u, e[i].x, e[i].y);
          else mma_16816(acc[i & 3], xf[XS * ii], xf[XS * ii + 1], xf[XS * ii + 2], xf[XS * ii + 3], e[i].x, e[i].y);
        }
      }
    } else {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {   // two halves of 4 lookups keep the register count down
        uint4 e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) e[i] = lds128(img + (idx_at<IB>(w, 4 * hf + i, cmax) << ENTRY_SHIFT), epoch);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ii = 4 * hf + i;
          if constexpr (FORM == 2) {
            mma_16816(acc[(2 * i) & 3], xf[XS * 2 * ii], 0u, xf[XS * 2 * ii + 1], 0u, e[i].x, e[i].y);
            mma_16816(acc[(2 * i + 1) & 3], xf[XS * (2 * ii + 1)], 0u, xf[XS * (2 * ii + 1) + 1], 0u, e[i].z, e[i].w);
          } else {
            mma_16816(acc[(2 * i) & 3], xf[XS * 2 * ii], xf[XS * 2 * ii + 1], xf[XS * 2 * ii + 2], xf[XS * 2 * ii + 3], e[i].x, e[i].y);
            mma_16816(acc[(2 * i + 1) & 3], xf[XS * (2 * ii + 1)], xf[XS * (2 * ii + 1) + 1], xf[XS * (2 * ii + 1) + 2],
                      xf[XS * (2 * ii + 1) + 3], e[i].z, e[i].w);
          }
        }
      }
    }
  }
}

// V: sub-vector length (4 or 8); IB: index bytes (1 or 2; 2 only with V = 8);
// FORM: 1 (M <= 4), 2 (M <= 8), 3 (M <= 16; form 2 with batch rows g+8 live);
// REPL: codebook image replicated to fill 128-byte lines (conflict-free) or stored once.
//
// An item is rl tiles side by side (8*SU rows each) of one K chunk; a CTA works through a contiguous
// range of items, in batches of up to `batch` items of one chunk that touch at most `nslots`
// consecutive codebook groups.  A batch ends with ONE block-wide barrier and a fixed-order sum of the
// warps' partial tiles (double-buffered, so the next batch's lookups run meanwhile).
//
// Shared memory (1024-aligned):  [warp rings][mbarriers][image slot 0][image slot 1][partial tiles x2][running sums]
template <int V, int IB, int FORM, bool REPL>
__global__ void __launch_bounds__(Geo<V, IB, FORM>::NT, (FORM == 1) ? 2 : 1)
vq_decode_kernel(const __grid_constant__ CUtensorMap idx_map, const DecodeParams p) {
  using G = Geo<V, IB, FORM>;
  constexpr int NW = G::NW, NT = G::NT, KS = G::KS, TK = G::TK, SLABB = G::SLABB, TB = G::TB, SU = G::SU;
  constexpr int STAGE = G::STAGE, XR = G::XR, W64 = G::W64;
  constexpr int ENTRY_LOG2 = (V == 4) ? 3 : 4;
  constexpr int REP_LOG2 = REPL ? (7 - ENTRY_LOG2) : 0;  // replicas fill a 128-byte line, or none at all
  constexpr int ENTRY_SHIFT = ENTRY_LOG2 + REP_LOG2;
  constexpr int PIECES = TK / 64;                        // 64-K pieces per thread and unit
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_last[kMaxBatch];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - smem_u32(smem_raw));

  // the next kernel in the stream may be scheduled as soon as SMs have room (it waits as below before it
  // touches anything this kernel reads or writes)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // static contiguous partition of the items (chunk-major so X stays in registers); the host supplies
  // quotient and remainder
  const int bid = blockIdx.x;
  int it0 = bid * p.items_q + min(bid, p.items_r);
  int it1 = it0 + p.items_q + (bid < p.items_r ? 1 : 0);
  if (it1 <= it0) return;
  // items of one chunk this CTA walks: all of them (its range then runs over chunks and items, chunk-major), or
  // its own range once per chunk
  int div = p.nrbg, off = 0;
  if (p.row_owned) {
    off = it0;
    div = it1 - it0;
    it0 = 0;
    it1 = div * p.nchunks;
  }
  const int nitems = it1 - it0;
  const int r_end = off + div;

  // warp role inside a chunk: (slice, row lane)
  const int nsl_full = min(NW, p.nslices);
  const int wsl = warp % nsl_full;
  const int wrl = warp / nsl_full;
  const bool role_ok = wrl < p.rl;
  const int S = p.stages;
  const uint32_t my_ring = base + static_cast<uint32_t>(warp * S) * STAGE;
  const uint32_t my_bars = base + p.bar_offset + static_cast<uint32_t>(warp * S) * 8;

  // ---- this warp's tile stream: requests run up to S tiles ahead of use -------------------------------
  int p_left = nitems;            // items not yet looked at by the requester
  int p_chunk = 0, p_rbg = off + it0;   // the next one
  if (it0 >= div) {                     // only when (chunk, item) pairs are dealt out and this range starts in a later chunk
    p_chunk = it0 / div;
    p_rbg = it0 - p_chunk * div;
  }
  const int first_chunk = p_chunk, first_rbg = p_rbg;
  // a chunk is (residual stage, chunk of K): chunk = stage * kchunks + kchunk
  int p_stg = (p.kchunks > 0 && p_chunk >= p.kchunks) ? p_chunk / p.kchunks : 0;
  int p_kchunk = p_chunk - p_stg * p.kchunks;
  int p_stage = 0, in_flight = 0;
  auto request_tiles = [&]() {
    while (p_left > 0 && in_flight < S) {
      const int slice = p_kchunk * NW + wsl;
      if (role_ok && slice < p.nslices) {
        if (lane == 0) {
          const uint32_t bar = my_bars + p_stage * 8;
          tc::mbar_expect_tx(bar, STAGE);
          tc::tma_load_2d(my_ring + p_stage * STAGE, &idx_map, slice * SLABB,
                          p_stg * p.stage_rows + (p_rbg * p.rl + wrl) * (8 * SU), bar);
        }
        p_stage = (p_stage + 1 == S) ? 0 : p_stage + 1;
        ++in_flight;
      }
      --p_left;
      if (++p_rbg == r_end) {
        p_rbg = off;
        ++p_chunk;
        if (++p_kchunk == p.kchunks) { p_kchunk = 0; ++p_stg; }
      }
    }
  };
  if (lane == 0) {
    for (int s = 0; s < S; ++s) tc::mbar_init(my_bars + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  request_tiles();
  int c_stage = 0;
  uint32_t c_parity = 0;

  const uint32_t img_bytes = static_cast<uint32_t>(p.C) << ENTRY_SHIFT;
  const uint32_t cmax = static_cast<uint32_t>(p.C - 1);
  // this lane's replica inside an image (32-bit shared address of slot 0)
  const uint32_t img_lane = base + p.img_offset + ((lane & ((1 << REP_LOG2) - 1)) << ENTRY_LOG2);
  uint32_t epoch = 0;
  float* part = reinterpret_cast<float*>(smem + p.part_offset);       // [2][batch][NW][SU][M][8]
  float* accbuf = reinterpret_cast<float*>(smem + p.acc_offset);      // [item - off][rl][SU][M][8], row-owned mode
  const int item_floats = SU * p.M * 8;

  // Builds the images of up to two groups (no barriers inside).  All global loads go out before the first
  // store, so a build costs one round trip to memory.  Replicated image: a thread loads one entry and writes
  // its copies, starting at a copy that depends on the entry so that a quarter warp's 16-byte stores fall into
  // different banks.
  using EntryT = typename std::conditional<V == 4, uint2, uint4>::type;
  auto build_images = [&](int group_a, bool need_a, int group_b, bool need_b) {
    unsigned char* img_a = smem + p.img_offset;
    unsigned char* img_b = img_a + img_bytes;
    const EntryT* src_a = reinterpret_cast<const EntryT*>(p.cb) + static_cast<size_t>(group_a) * p.C;
    const EntryT* src_b = reinterpret_cast<const EntryT*>(p.cb) + static_cast<size_t>(group_b) * p.C;
    if constexpr (REPL) {
      auto put = [&](unsigned char* img, int c, const EntryT& e) {
        uint4 q;
        if constexpr (V == 4) q = make_uint4(e.x, e.y, e.x, e.y); else q = e;
#pragma unroll
        for (int r = 0; r < 8; ++r) *reinterpret_cast<uint4*>(img + c * 128 + (((r + c) & 7) << 4)) = q;
      };
      for (int c = tid; c < p.C; c += NT) {
        EntryT ea{}, eb{};
        if (need_a) ea = __ldg(src_a + c);
        if (need_b) eb = __ldg(src_b + c);
        if (need_a) put(img_a, c, ea);
        if (need_b) put(img_b, c, eb);
      }
    } else {
      for (int pass = 0; pass < 2; ++pass) {
        if (!(pass ? need_b : need_a)) continue;
        const EntryT* src = pass ? src_b : src_a;
        EntryT* img = reinterpret_cast<EntryT*>(pass ? img_b : img_a);
        for (int c0 = 0; c0 < p.C; c0 += 8 * NT) {
          EntryT e[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * NT + tid;
            if (c < p.C) e[j] = __ldg(src + c);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * NT + tid;
            if (c < p.C) img[c] = e[j];
          }
        }
      }
    }
  };

  uint32_t xf[XR];
  // X fragment registers of this thread for its quarter of the warp's slice in `chunk`, straight from global
  // memory (L2) in register order.
  auto load_x = [&](int chunk, bool active) {
    const int kt = (chunk * NW + wsl) * KS + t4 * TK;
    if constexpr (FORM == 1) {
      // B fragment of column g = (batch row g/2, pair selector g%2): for each group q of 8 K values,
      // register 0 = pair {0-1} or {2-3}, register 1 = pair {4-5} or {6-7}
      const int m = g >> 1, h = g & 1;
      const bool live = active && m < p.M;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(p.x + static_cast<size_t>(live ? m : 0) * p.K + (live ? kt : 0)) + h;
#pragma unroll
      for (int q = 0; q < TK / 8; ++q) {
        uint32_t v0 = 0u, v1 = 0u;
        if (live) { v0 = __ldg(src + 4 * q); v1 = __ldg(src + 4 * q + 2); }
        xf[2 * q] = v0;
        xf[2 * q + 1] = v1;
      }
    } else {
      // A fragment rows g (and g+8): 4 consecutive K values per MMA, so 16 bytes of a row are the row's registers
      // of two MMAs, in order.  The warp reads its slice of eight batch rows with coalesced 16-byte loads (one
      // row = 512 contiguous bytes per instruction), passes them through 4 KiB of its own in shared memory and
      // every thread picks up the 128 bytes of row g that belong to its quarter of the slice.  Chunks of 16
      // bytes are placed at (c & 7) ^ ((c >> 3) & 3) ^ ((row & 1) << 2) within their 128-byte line, which makes
      // both the stores and the loads conflict-free.
      const uint32_t sx = base + p.part_offset + warp * 4096;
      const __half* xs = p.x + (chunk * NW + wsl) * KS + lane * 8;
#pragma unroll
      for (int pass = 0; pass < (FORM == 3 ? 2 : 1); ++pass) {
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = pass * 8 + i;
          v[i] = make_uint4(0u, 0u, 0u, 0u);
          if (active && r < p.M) v[i] = __ldg(reinterpret_cast<const uint4*>(xs + static_cast<size_t>(r) * p.K));
        }
        __syncwarp();   // the previous pass has been read
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t c = (lane & ~7u) | ((lane ^ (lane >> 3) ^ ((i & 1) << 2)) & 7u);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sx + i * 512 + (c << 4)), "r"(v[i].x), "r"(v[i].y),
                       "r"(v[i].z), "r"(v[i].w) : "memory");
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < TK / 8; ++j) {
          const uint32_t lc = t4 * 8 + j;
          const uint32_t c = (lc & ~7u) | ((lc ^ (lc >> 3) ^ ((g & 1) << 2)) & 7u);
          const uint4 q = lds128_tile(sx + g * 512 + (c << 4));
          if constexpr (FORM == 3) {
            xf[8 * j + pass] = q.x; xf[8 * j + 2 + pass] = q.y; xf[8 * j + 4 + pass] = q.z; xf[8 * j + 6 + pass] = q.w;
          } else {
            xf[4 * j + 0] = q.x; xf[4 * j + 1] = q.y; xf[4 * j + 2] = q.z; xf[4 * j + 3] = q.w;
          }
        }
      }
    }
  };

  int loaded_kchunk = -1;
  int slot_group0 = -1, slot_group1 = -1;   // which group each image slot holds
  bool active = false;
  bool first_batch = true;
  int parity = 0;

  int seq = 0;
  int chunk = first_chunk;
  int rbg = first_rbg;
  int stg = (chunk >= p.kchunks) ? chunk / p.kchunks : 0;   // residual stage and K chunk of `chunk`
  int kchunk = chunk - stg * p.kchunks;
  while (seq < nitems) {
    // ---- the batch: items [seq, seq + cnt) = row block groups [rbg, rbg + cnt) of `chunk` ----------------
    const int group_in_stage = rbg / p.ipg;
    const int gpos = rbg - group_in_stage * p.ipg;
    const int group = stg * p.ngroups + group_in_stage;    // codebooks of all stages, stage-major
    int cnt = min(min(p.batch, nitems - seq), min(r_end - rbg, p.nslots * p.ipg - gpos));
    const int g_first = group;
    const int g_last = group + ((gpos + cnt - 1 >= p.ipg) ? 1 : 0);   // a batch touches at most two groups
    {
      const bool need0 = (p.nslots == 1) ? (slot_group0 != g_first)
                                         : ((((g_first & 1) == 0) && slot_group0 != g_first) ||
                                            (((g_last & 1) == 0) && slot_group0 != g_last));
      const bool need1 = (p.nslots == 2) && ((((g_first & 1) == 1) && slot_group1 != g_first) ||
                                             (((g_last & 1) == 1) && slot_group1 != g_last));
      if (need0 || need1) {
        if (!first_batch) __syncthreads();   // everyone is done looking up in the old images
        if (need0) slot_group0 = (p.nslots == 1 || (g_first & 1) == 0) ? g_first : g_last;
        if (need1) slot_group1 = ((g_first & 1) == 1) ? g_first : g_last;
        build_images(need0 ? slot_group0 : 0, need0, need1 ? slot_group1 : 0, need1);
        __syncthreads();
        asm volatile("add.u32 %0, %0, 1;" : "+r"(epoch));
      }
    }

    // Everything above reads only the weights (indices, codebooks).  X, Y and the workspace belong to the
    // stream's order: when the launch was made with programmatic stream serialisation this kernel may have
    // started while its predecessor was still running, and waits here for it to complete.
    if (first_batch) asm volatile("griddepcontrol.wait;" ::: "memory");
    first_batch = false;
    if (kchunk != loaded_kchunk) {
      // forms 2/3 pass X through the memory of the partial tiles: nobody may still be summing the last batch
      if (FORM != 1 && loaded_kchunk >= 0) __syncthreads();
      active = role_ok && (kchunk * NW + wsl) < p.nslices;
      load_x(kchunk, active);
      if (FORM != 1) __syncthreads();   // ... and nobody writes partial tiles before every warp has its X
      loaded_kchunk = kchunk;
    }

    float* pb = part + static_cast<size_t>(parity) * (p.batch * NW * item_floats);
    parity ^= 1;
    if (active) {
      for (int s = 0; s < cnt; ++s) {
        // image of this item's group
        const int grp = group + ((gpos + s >= p.ipg) ? 1 : 0);
        const uint32_t img_s = img_lane + ((p.nslots == 2 && (grp & 1)) ? img_bytes : 0u);
        tc::mbar_wait(my_bars + c_stage * 8, c_parity, p.status, DS_TMA_FULL_TIMEOUT);
        const uint32_t tile = my_ring + c_stage * STAGE;
        float* mine = pb + static_cast<size_t>(s * NW + warp) * item_floats;
#pragma unroll
        for (int j = 0; j < SU; ++j) {
          // this thread's TB index bytes of row r of the tile, through the tile's swizzle
          uint32_t w[TB / 4];
          const int r = j * 8 + g;
          if constexpr (SLABB == 128) {
            const uint32_t row = tile + r * 128;
            const uint4 a = lds128_tile(row + (((2 * t4) ^ g) << 4));
            const uint4 b = lds128_tile(row + (((2 * t4 + 1) ^ g) << 4));
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
          } else if constexpr (SLABB == 64) {
            const uint4 a = lds128_tile(tile + r * 64 + ((t4 ^ ((g >> 1) & 3)) << 4));
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
          } else {
            const uint2 a = lds64_tile(tile + r * 32 + (((t4 >> 1) ^ ((g >> 2) & 1)) << 4) + (t4 & 1) * 8);
            w[0] = a.x; w[1] = a.y;
          }
          float ch[4][4];   // four independent accumulation chains, summed in a fixed order
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) ch[a][c] = 0.f;
#pragma unroll
          for (int pc = 0; pc < PIECES; ++pc)
            piece_mma<V, IB, FORM, ENTRY_SHIFT>(ch, w + pc * W64, xf + pc * (XR / PIECES), img_s, epoch, cmax);
          float acc[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[c] = (ch[0][c] + ch[1][c]) + (ch[2][c] + ch[3][c]);
          // this warp's partial tile of the unit: [m][8 rows]
          float* dst = mine + j * p.M * 8;
          if constexpr (FORM == 1) {
            if (t4 < p.M) dst[t4 * 8 + g] = acc[0] + acc[3];
          } else {
            // acc = D[batch g][rows 2t, 2t+1], D[batch g+8][rows 2t, 2t+1]
            if (g < p.M) *reinterpret_cast<float2*>(dst + g * 8 + 2 * t4) = make_float2(acc[0], acc[1]);
            if (FORM == 3 && g + 8 < p.M) *reinterpret_cast<float2*>(dst + (g + 8) * 8 + 2 * t4) = make_float2(acc[2], acc[3]);
          }
        }
        // the tile has been read by every lane: its place in the ring takes the next request
        __syncwarp();
        --in_flight;
        if (++c_stage == S) { c_stage = 0; c_parity ^= 1; }
        request_tiles();
      }
    } else {
      // warps without a slice in this chunk (or without a row lane) still step the requester past the batch
      request_tiles();
    }
    __syncthreads();

    // fixed-order sum over the slices of the chunk, one thread per output
    const int nsl = min(NW, p.nslices - kchunk * NW);
    const int outs = cnt * p.rl * item_floats;
    const bool split = p.nchunks > 1 && !p.row_owned;
    const bool carry = p.nchunks > 1 && p.row_owned;   // running sums over the chunks in shared memory
    for (int o = tid; o < outs; o += NT) {
      // o = ((s * rl + lr) * SU + j) * M * 8 + m * 8 + r8, taken apart with host-made reciprocals
      const int r8 = o & 7;
      const int t = o >> 3;
      const int tj = p.inv_m ? __umulhi(static_cast<unsigned>(t), p.inv_m) : t;   // t / M = (s * rl + lr) * SU + j
      const int m = t - tj * p.M;
      const int j = tj & (SU - 1);
      const int tl = tj / SU;                                             // s * rl + lr
      const int s = p.inv_rl ? __umulhi(static_cast<unsigned>(tl), p.inv_rl) : tl;
      const int lr = tl - s * p.rl;
      const int row = (((rbg + s) * p.rl + lr) * SU + j) * 8 + r8;
      const float* src = pb + static_cast<size_t>(s * NW + lr * nsl_full) * item_floats + (j * p.M + m) * 8 + r8;
      float sum = 0.f;
      if (nsl == NW) {
#pragma unroll
        for (int sl = 0; sl < NW; ++sl) sum += src[sl * item_floats];
      } else {
        for (int sl = 0; sl < nsl; ++sl) sum += src[sl * item_floats];
      }
      if (row >= p.N) continue;
      if (carry) {
        // place of this output in the CTA's accumulator: the same for every chunk
        float* a = accbuf + (static_cast<size_t>(rbg + s - off) * p.rl + lr) * item_floats + (j * p.M + m) * 8 + r8;
        if (chunk > 0) sum += *a;
        if (chunk + 1 < p.nchunks) { *a = sum; continue; }
      } else if (split) {
        __stcg(p.ws_partial + (static_cast<size_t>(chunk) * p.M + m) * p.N + row, sum);
        continue;
      }
      const __half h = __float2half_rn(sum);
      const size_t o_off = static_cast<size_t>(m) * p.ld_y + row;
      p.y[o_off] = h;
      for (int pq = 0; pq < p.n_peers; ++pq) p.peer_y[pq][o_off] = h;
    }
    if (split) {
      // split-K: the CTA that brings an item's counter to nchunks sums the chunks in chunk order
      __threadfence();
      __syncthreads();
      if (tid < cnt) {
        const int old = atomicAdd(p.ws_counter + rbg + tid, 1);
        const int last = (old == p.nchunks - 1);
        if (last) p.ws_counter[rbg + tid] = 0;  // leave the counter zero for the next call
        s_last[tid] = last;
      }
      __syncthreads();
      __threadfence();
      for (int o = tid; o < outs; o += NT) {
        const int r8 = o & 7;
        const int t = o >> 3;
        const int tj = p.inv_m ? __umulhi(static_cast<unsigned>(t), p.inv_m) : t;
        const int m = t - tj * p.M;
        const int j = tj & (SU - 1);
        const int tl = tj / SU;
        const int s = p.inv_rl ? __umulhi(static_cast<unsigned>(tl), p.inv_rl) : tl;
        const int lr = tl - s * p.rl;
        if (!s_last[s]) continue;
        const int row = (((rbg + s) * p.rl + lr) * SU + j) * 8 + r8;
        if (row >= p.N) continue;
        float sum = 0.f;
        for (int c = 0; c < p.nchunks; ++c)
          sum += __ldcg(p.ws_partial + (static_cast<size_t>(c) * p.M + m) * p.N + row);
        const __half h = __float2half_rn(sum);
        const size_t o_off = static_cast<size_t>(m) * p.ld_y + row;
        p.y[o_off] = h;
        for (int pq = 0; pq < p.n_peers; ++pq) p.peer_y[pq][o_off] = h;
      }
      __syncthreads();  // s_last is rewritten by the next batch
    }

    seq += cnt;
    rbg += cnt;
    if (rbg == r_end) {
      rbg = off;
      ++chunk;
      if (++kchunk == p.kchunks) { kchunk = 0; ++stg; }
    }
  }
}

// Full replication (16 or 8 copies fill a 128-byte line) when the image fits the budget, else none.
int pick_rep_log2(int v, int C, size_t budget) {
  const int rep = (v == 4) ? 4 : 3;
  return (static_cast<size_t>(C) * 2 * v << rep) <= budget ? rep : 0;
}

int device_sms() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

struct Plan {
  DecodeParams d;
  int form, nw, ks, su, slabb, stage, rep_log2;
  size_t smem;
  int grid;
  size_t ws_bytes;   // split-K scratch this plan needs (0 if none)
};

// Everything the launch needs except pointers into a workspace.  Returns false for shapes outside the kernel.
bool make_plan(const Problem& p, Plan& pl) {
  if (p.M < 1 || p.M > 16) return false;
  if (!(p.v == 4 || p.v == 8)) return false;
  if (!(p.idx_bytes == 1 || (p.idx_bytes == 2 && p.v == 8))) return false;
  if (p.K % 256 != 0 || p.N % 8 != 0 || p.K == 0 || p.N == 0) return false;
  const bool single = p.rows_per_cb >= p.N;
  if (p.idx_bytes == 1 && p.C > 256) return false;
  if (p.C > 65536 || p.C < 1) return false;
  if (reinterpret_cast<uintptr_t>(p.x) % 16 || reinterpret_cast<uintptr_t>(p.idx) % 16 ||
      reinterpret_cast<uintptr_t>(p.cb) % 16)
    return false;
  const size_t entry = static_cast<size_t>(2) * p.v;
  if (p.C * entry > 160 * 1024) return false;
  DecodeParams& d = pl.d;
  d = DecodeParams{};
  // form 1 needs whole 512-wide slices; other K (multiples of 256) take the two-row-halves form, which holds M <= 8
  pl.form = (p.M <= 4 && p.K % 512 == 0) ? 1 : (p.M <= 8 ? 2 : 3);
  pl.nw = pl.form == 1 ? 8 : 16;
  pl.ks = pl.form == 1 ? 512 : 256;
  pl.slabb = pl.ks / p.v * p.idx_bytes;
  pl.su = pl.slabb >= 128 ? 1 : 2;
  pl.stage = 8 * pl.su * pl.slabb;
  const int tile_rows = 8 * pl.su;
  if (!single && p.rows_per_cb % tile_rows != 0) return false;
  d.nslices = p.K / pl.ks;
  const int wstages = p.n_stages > 1 ? p.n_stages : 1;   // residual stages of the weights
  if (wstages > 8) return false;
  d.kchunks = (d.nslices + pl.nw - 1) / pl.nw;
  d.nchunks = d.kchunks * wstages;
  d.stage_rows = p.N;
  const int nsl_full = d.nslices < pl.nw ? d.nslices : pl.nw;
  const int tiles = (p.N + tile_rows - 1) / tile_rows;
  const int tiles_per_group = single ? tiles : (p.rows_per_cb / tile_rows);
  int rl = pl.nw / nsl_full;
  while (rl > 1 && (tiles % rl != 0 || tiles_per_group % rl != 0)) --rl;
  d.rl = rl;
  d.nrbg = tiles / rl;
  d.ipg = tiles_per_group / rl;
  d.ngroups = single ? 1 : (p.N + p.rows_per_cb - 1) / p.rows_per_cb;
  // residual stages: the tiles of stage s are found s * N rows further down, so N must hold whole tiles
  if (wstages > 1 && p.N % tile_rows != 0) return false;

  const int sms = device_sms();
  // what is dealt out over the CTAs: (chunk, item) pairs, or the items of one chunk in the row-owned mode.
  // Row-owned walk of the K chunks: worth it when there are several chunks and enough items that an even split of
  // them over the SMs is balanced (at least six per CTA), and when the running sums of a CTA's rows fit shared memory.
  const int item_floats = pl.su * p.M * 8;
  const size_t item_bytes = static_cast<size_t>(pl.nw) * item_floats * sizeof(float);   // partial tiles of one item
  pl.rep_log2 = pick_rep_log2(p.v, p.C, 64 * 1024);
  const size_t img_bytes = static_cast<size_t>(p.C) * entry << pl.rep_log2;
  const size_t budget = pl.form == 1 ? 112 * 1024 : 220 * 1024;   // form 1: two launches side by side on an SM
  // a second resident image lets a batch straddle a group boundary; only where it leaves room for the rest
  const size_t rest_min = 2 * item_bytes + static_cast<size_t>(pl.nw) * (4 * pl.stage + (pl.form != 1 ? 4096 : 0)) + 8192;
  d.nslots = (!single && 2 * img_bytes + (rest_min > 48 * 1024 ? rest_min : 48 * 1024) <= budget) ? 2 : 1;
  size_t acc_bytes = 0;
  d.row_owned = 0;
  if (d.nchunks > 1 && d.nrbg >= 6 * sms) {
    const int per_cta = (d.nrbg + sms - 1) / sms;
    const size_t need = static_cast<size_t>(per_cta) * rl * item_floats * sizeof(float);
    if (need + d.nslots * img_bytes + 2 * item_bytes + static_cast<size_t>(pl.nw) * 2 * pl.stage + 4096 <= 220 * 1024) {
      d.row_owned = 1;
      acc_bytes = need;
    }
  }
  const long long items = d.row_owned ? d.nrbg : static_cast<long long>(d.nchunks) * d.nrbg;
  pl.grid = static_cast<int>(items < sms ? items : sms);
  d.items_q = static_cast<int>(items / pl.grid);
  d.items_r = static_cast<int>(items % pl.grid);
  const int per_cta_items = d.items_q + (d.items_r ? 1 : 0);

  // shared memory: images and running sums are fixed; the rest goes to reduction batches and tiles in flight
  const size_t fixed = d.nslots * img_bytes + acc_bytes + static_cast<size_t>(pl.nw) * 8 * 8 + 2048;
  if (fixed + 2 * item_bytes + static_cast<size_t>(pl.nw) * (2 * pl.stage + (pl.form != 1 ? 4096 : 0)) > 224 * 1024) return false;
  const size_t total_budget =
      (acc_bytes || fixed + 2 * item_bytes + static_cast<size_t>(pl.nw) * 2 * pl.stage > budget) ? 224 * 1024 : budget;
  // batches of equal size: as few as kMaxBatch items per batch allow, within half of the memory that is left
  int batch = per_cta_items < 1 ? 1 : per_cta_items;
  for (int nb = 1; batch > kMaxBatch || (batch > 1 && 2 * batch * item_bytes > (total_budget - fixed) / 2); ++nb)
    batch = (per_cta_items + nb) / (nb + 1);
  if (batch < 1) batch = 1;
  d.batch = batch;
  size_t part_bytes = 2 * batch * item_bytes;
  // forms 2/3 pass the X fragments through this memory, 4 KiB per warp
  if (pl.form != 1 && part_bytes < static_cast<size_t>(pl.nw) * 4096) part_bytes = static_cast<size_t>(pl.nw) * 4096;
  d.inv_m = p.M > 1 ? static_cast<unsigned>((0x100000000ULL + p.M - 1) / p.M) : 0u;
  d.inv_rl = rl > 1 ? static_cast<unsigned>((0x100000000ULL + rl - 1) / rl) : 0u;
  int stages = static_cast<int>((total_budget - fixed - part_bytes) / (static_cast<size_t>(pl.nw) * pl.stage));
  if (stages > 8) stages = 8;
  if (stages < 2) return false;
  d.stages = stages;
  const size_t ring = static_cast<size_t>(pl.nw) * stages * pl.stage;   // multiple of 1024 (nw*stage is)
  d.bar_offset = static_cast<int>(ring);
  d.img_offset = static_cast<int>((ring + static_cast<size_t>(pl.nw) * stages * 8 + 127) & ~static_cast<size_t>(127));
  d.part_offset = static_cast<int>(d.img_offset + d.nslots * img_bytes);
  d.acc_offset = static_cast<int>(d.part_offset + part_bytes);
  pl.smem = d.acc_offset + acc_bytes + 1024;   // + alignment slack
  if (p.idx_bytes == 1 && p.C < 256) {
    // an 8-bit index beyond a small codebook (malformed input) must still address inside the block's shared
    // memory: room for 256 entries behind the last image slot's base
    const size_t reach = d.img_offset + (d.nslots - 1) * img_bytes + (img_bytes / p.C) * 256 + 1024;
    if (pl.smem < reach) pl.smem = reach;
  }
  if (pl.smem > 227 * 1024) return false;

  pl.ws_bytes = 0;
  if (d.nchunks > 1 && !d.row_owned) {
    if (static_cast<size_t>(d.nrbg) * sizeof(int) > kCounterBytes) return false;
    pl.ws_bytes = kCounterBytes + static_cast<size_t>(d.nchunks) * p.M * p.N * sizeof(float);
  }
  d.x = p.x; d.cb = p.cb; d.y = p.y;
  d.M = p.M; d.N = p.N; d.K = p.K; d.C = p.C;
  d.ld_y = p.ld_y;
  d.n_peers = p.n_peers;
  for (int i = 0; i < 8; ++i) d.peer_y[i] = p.peer_y[i];
  return true;
}

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

// The index matrix as bytes [N][J * idx_bytes]; one box = one warp tile, swizzled over its row length.
bool make_idx_map(CUtensorMap* map, const Problem& p, const Plan& pl) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(p.K / p.v) * p.idx_bytes;
  const cuuint64_t dims[2] = {row_bytes, static_cast<cuuint64_t>(p.N) * (p.n_stages > 1 ? p.n_stages : 1)};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(pl.slabb), static_cast<cuuint32_t>(8 * pl.su)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = pl.slabb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                                : (pl.slabb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(p.idx), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

using KernelT = void (*)(const CUtensorMap, const DecodeParams);

KernelT pick_kernel(const Problem& p, const Plan& pl) {
  KernelT k = nullptr;
#define VQG_PICK(V_, IB_)                                                                                \
  if (p.v == V_ && p.idx_bytes == IB_) {                                                                 \
    if (pl.rep_log2 > 0)                                                                                 \
      k = pl.form == 1 ? vq_decode_kernel<V_, IB_, 1, true>                                              \
                       : (pl.form == 2 ? vq_decode_kernel<V_, IB_, 2, true> : vq_decode_kernel<V_, IB_, 3, true>); \
    else                                                                                                 \
      k = pl.form == 1 ? vq_decode_kernel<V_, IB_, 1, false>                                             \
                       : (pl.form == 2 ? vq_decode_kernel<V_, IB_, 2, false> : vq_decode_kernel<V_, IB_, 3, false>); \
  }
  VQG_PICK(4, 1) VQG_PICK(8, 1) VQG_PICK(8, 2)
#undef VQG_PICK
  return k;
}

// One launch of the planned kernel; `dependent` adds programmatic stream serialisation (set-up, the codebook image
// and the first index tiles of this launch overlap the tail of the kernel before it in the stream).
int launch_planned(const Problem& p, Plan& pl, bool dependent, cudaStream_t s) {
  CUtensorMap map;
  if (!make_idx_map(&map, p, pl)) return VQG_ERR_LAUNCH;
  KernelT k = pick_kernel(p, pl);
  if (!k) return VQG_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pl.smem));
  if (e != cudaSuccess) return VQG_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pl.grid));
  cfg.blockDim = dim3(static_cast<unsigned>(pl.nw * 32));
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, k, map, pl.d);
  count_launch();
  return cuda_status(e == cudaSuccess ? cudaGetLastError() : e);
}

}  // namespace

bool decode_supported(const Problem& p) {
  Plan pl;
  return make_plan(p, pl);
}

size_t decode_workspace_bytes(const Problem& p) {
  Plan pl;
  return make_plan(p, pl) ? pl.ws_bytes : 0;
}

int launch_decode(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s) {
  Plan pl;
  if (!make_plan(p, pl)) return VQG_ERR_UNSUPPORTED;
  if (pl.ws_bytes) {
    if (ws == nullptr || ws_bytes < pl.ws_bytes) return VQG_ERR_WORKSPACE;
    pl.d.ws_counter = static_cast<int*>(ws);
    pl.d.ws_partial = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + kCounterBytes);
  }
  pl.d.status = device_status_ptr();
  // the weight-only prologue may run beside the kernel ahead on the stream -- unless that kernel wrote the weights
  return launch_planned(p, pl, /*dependent=*/!take_weights_written(s), s);
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

// Device address of the static scratch on the current device; looked up on the first call per device.  That
// first lookup is also what makes the CUDA runtime load this module onto the device, array included.
int static_scratch_ptr(unsigned char** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return VQG_ERR_NO_DEVICE;
  if (dev < 0 || dev >= 64) return VQG_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    unsigned char* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e == cudaErrorMemoryAllocation) {
      cudaGetLastError();
      return VQG_ERR_NO_MEMORY;
    }
    if (e != cudaSuccess || ptr == nullptr) return VQG_ERR_LAUNCH;
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return VQG_OK;
}
}  // namespace

int launch_decode_static(const Problem& p, cudaStream_t s) {
  Plan pl;
  if (!make_plan(p, pl)) return VQG_ERR_UNSUPPORTED;
  if (pl.ws_bytes > kStaticScratchBytes) return VQG_ERR_TOO_LARGE;
  unsigned char* scratch = nullptr;
  const int st = static_scratch_ptr(&scratch);
  if (st != VQG_OK) return st;
  if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
  if (pl.ws_bytes) {
    // the array keeps whatever the previous call left: the arrival counters must start at zero
    if (cudaMemsetAsync(scratch, 0, static_cast<size_t>(pl.d.nrbg) * sizeof(int), s) != cudaSuccess) return VQG_ERR_LAUNCH;
    pl.d.ws_counter = reinterpret_cast<int*>(scratch);
    pl.d.ws_partial = reinterpret_cast<float*>(scratch + kCounterBytes);
  }
  pl.d.status = device_status_ptr();
  return launch_planned(p, pl, /*dependent=*/false, s);
}

}  // namespace vqg
