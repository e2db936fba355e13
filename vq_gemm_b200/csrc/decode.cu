// Memory-bound VQ-GEMM for M <= 16 (decode / small batch), sm_100a.
//
// The problem is a GEMV-like stream over the index matrix: every index is read once from HBM
// and costs one shared-memory codebook lookup.  The kernel is persistent (one 512-thread CTA per
// SM) and works on items of 16 output rows x up to 4096 K values:
//
//   * indices are streamed with 64-/128-bit loads straight into registers, one batch (2-3 items)
//     ahead of use, so tens of KiB per SM are in flight;
//   * the codebook of the item's group sits in shared memory as a REPLICATED image: entry c,
//     replica r at byte  c*(R*2v) + r*2v , lane uses replica lane % R.  With R = 64/v
//     (C <= 256) a warp-wide lookup touches every bank exactly once per wavefront;
//   * looked-up entries go into mma.sync.m16n8k16 operand registers AS THEY ARRIVE -- no
//     conversion, shuffle or register move -- and accumulation is fp32 in the tensor core.  Every
//     thread (g, t) of a warp owns weight row n0+g and the 64 K values [64t, 64t+64) of the
//     warp's 256-wide K slice.  Two operand arrangements:
//       form 1 (M <= 4)  16 bytes of codebook data (one v=8 entry, or two consecutive v=4 entries)
//         are the 4 registers of an A fragment: MMA row g sees K pairs {0-1, 4-5} of them, MMA row
//         g+8 sees pairs {2-3, 6-7}.  X is the B operand with two columns per batch row m:
//         column 2m carries X for the pairs of row g, column 2m+1 those of row g+8, so that
//         y[n0+g][m] = D[g][2m] + D[g+8][2m+1].  One MMA per 16 codebook bytes.
//       form 2 (M <= 16) a v=4 entry (or half a v=8 entry) is the 2-register B fragment of
//         column g; X (batch rows g and g+8) is the A operand.  One MMA per 8 codebook bytes.
//     The X fragments are loaded once and stay in registers;
//   * each warp owns a 256-wide K slice; the 16 partial tiles of a CTA are summed in a fixed
//     order through shared memory (deterministic), one barrier per batch, and K > 4096 adds a
//     split-K step through a caller-provided workspace in which the last-arriving CTA of a row
//     block sums the chunks in chunk order (also deterministic).
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
  int nslots;          // resident codebook images (1 or 2)
  int items_q, items_r; // items per CTA: q, and one more for the first r CTAs
  int ipg;             // items per codebook group
  int lpo;             // lanes per output in the cross-warp reduction (power of two)
  int lpo_log2;
  int inv_m, inv_rl;   // ceil(65536 / M), ceil(65536 / rl): t / M == (t * inv_m) >> 16 for t < 4096
  int n_peers;
  __half* peer_y[8];
  // K > 4096 on matrices with many row blocks: a CTA owns a range of row blocks for ALL K chunks (items_q/r then
  // partition the row blocks), walks the chunks one after the other and keeps the running sums of its rows in
  // shared memory at byte offset acc_offset -- no partial sums in global memory, no counters, no hand-over.
  int row_owned;
  int acc_offset;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
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

template <int WORDS>
struct IdxRegs { uint32_t w[WORDS]; };

template <int WORDS>
__device__ __forceinline__ void load_idx(IdxRegs<WORDS>& r, const void* p) {
  if constexpr (WORDS == 2) {
    uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    r.w[0] = t.x; r.w[1] = t.y;
  } else {
    uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
    r.w[0] = t.x; r.w[1] = t.y; r.w[2] = t.z; r.w[3] = t.w;
  }
}

template <int IB>
__device__ __forceinline__ uint32_t idx_at(const uint32_t* w, int i) {
  if constexpr (IB == 1) return __byte_perm(w[i >> 2], 0, 0x4440 + (i & 3));
  else return __byte_perm(w[i >> 1], 0, (i & 1) ? 0x4432 : 0x4410);
}

// V: sub-vector length (4 or 8); IB: index bytes (1 or 2; 2 only with V = 8);
// FORM: 1 (M <= 4), 2 (M <= 8), 3 (M <= 16; form 2 with batch rows g+8 live);
// REPL: codebook image replicated to fill 128-byte lines (conflict-free) or stored once.
//
// Items are processed in batches of up to PFB consecutive items of one K chunk.  While a batch is
// being computed the index loads of the next batch are in flight; a batch ends with ONE block-wide
// barrier and a parallel, fixed-order reduction of the 16 warps' partial tiles.  Up to two codebook
// images (groups of even / odd number) are resident, so a batch may straddle a group boundary.
//
// Shared memory:  [image slot 0][image slot 1 (if it fits)][ X staging | reduction buffers ]
template <int V, int IB, int FORM, bool REPL>
__global__ void __launch_bounds__(kThreads, 1) vq_decode_kernel(const DecodeParams p) {
  constexpr int UB = (IB == 1 && V == 8) ? 8 : 16;  // index bytes per thread and 8-row unit (= 64 K values)
  constexpr int WORDS = UB / 4;
  constexpr int NIDX = UB / IB;                      // indices per thread and unit
  constexpr int ENTRY_LOG2 = (V == 4) ? 3 : 4;
  constexpr int REP_LOG2 = REPL ? (7 - ENTRY_LOG2) : 0;  // replicas fill a 128-byte line, or none at all
  constexpr int ENTRY_SHIFT = ENTRY_LOG2 + REP_LOG2;
  // items per batch: every batch ends with two barriers, the cross-warp reduction and (K > 4096) the split-K
  // hand-over, so large matrices want long batches; with 16-byte entries the index registers are few
  constexpr int PFB = (FORM == 1) ? 6 : (FORM == 2 ? (V == 8 ? 6 : 3) : (V == 8 ? 4 : 2));
  constexpr int XR = (FORM == 1) ? 16 : (FORM == 2 ? 32 : 64);  // X fragment registers per thread
  constexpr int XSLOT = XR + 4;                      // staging words per thread (16-byte aligned, bank-spread)
  static_assert(NIDX * V == 64, "a thread-unit spans 64 K values");
  extern __shared__ __align__(16) unsigned char smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int J = p.K / V;

  const uint32_t img_bytes = static_cast<uint32_t>(p.C) << ENTRY_SHIFT;
  unsigned char* work = smem + static_cast<size_t>(p.nslots) * img_bytes;   // staging, then reduction buffers
  float* red = reinterpret_cast<float*>(work);                              // [2][kWarps][warp_stride]
  uint32_t* stage = reinterpret_cast<uint32_t*>(work);                      // [kWarps][32][XSLOT]
  const int unit_floats = p.M * 8;                           // [m][8 rows]
  const int warp_stride = PFB * 2 * unit_floats + 2;         // +2: slices land in different banks, 8-byte aligned
  __shared__ int s_last[PFB];

  // this lane's replica inside an image (32-bit shared address of slot 0)
  const uint32_t img_lane = smem_u32(smem) + ((lane & ((1 << REP_LOG2) - 1)) << ENTRY_LOG2);
  uint32_t epoch = 0;

  // static contiguous partition of the items (chunk-major so X stays in registers); the host supplies
  // quotient and remainder so that no 64-bit division runs on the device
  const int bid = blockIdx.x;
  int it_begin = bid * p.items_q + min(bid, p.items_r);
  int it_end = it_begin + p.items_q + (bid < p.items_r ? 1 : 0);
  // the next kernel in the stream may be scheduled as soon as SMs free up (it waits as below before it
  // touches anything this kernel reads or writes)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (it_end <= it_begin) return;
  // row blocks this CTA walks: all of them (items then run over chunks and row blocks, chunk-major), or its
  // own range once per chunk
  int r_begin = 0, r_end = p.nrbg;
  if (p.row_owned) {
    r_begin = it_begin;
    r_end = it_end;
    it_begin = 0;
    it_end = (r_end - r_begin) * p.nchunks;
  }
  float* accbuf = reinterpret_cast<float*>(smem + p.acc_offset);   // [row block - r_begin][rl][M][16], row-owned mode

  // warp role inside a chunk: (slice, row lane)
  const int nsl_full = min(kWarps, p.nslices);
  const int wsl = warp % nsl_full;
  const int wrl = warp / nsl_full;
  const bool role_ok = wrl < p.rl;
  const unsigned char* idx_lane = static_cast<const unsigned char*>(p.idx) +
      (static_cast<size_t>(wrl * 16 + g) * J + static_cast<size_t>(t4) * NIDX) * IB;
  const size_t row8_bytes = static_cast<size_t>(8) * J * IB;
  const size_t item_bytes = static_cast<size_t>(p.rl) * 16 * J * IB;   // rows of one item

  uint32_t xf[XR];
  int loaded_chunk = -1;
  int slot_group0 = -1, slot_group1 = -1;   // which group each image slot holds
  bool active = false;

  struct Batch { int cnt, chunk, rbg, gpos, group; };  // group/gpos: codebook group of the first item, position in it
  auto make_batch = [&](int it, int chunk, int rbg, int gpos, int group) {
    Batch b;
    b.chunk = chunk; b.rbg = rbg; b.gpos = gpos; b.group = group;
    int c = it_end - it;
    c = min(c, PFB);
    c = min(c, r_end - rbg);
    c = min(c, p.nslots * p.ipg - gpos);   // a batch touches at most `nslots` consecutive groups
    b.cnt = c > 0 ? c : 0;
    return b;
  };

  IdxRegs<WORDS> cur[PFB][2];
  auto issue_loads = [&](const Batch& b, IdxRegs<WORDS> (&dst)[PFB][2]) {
    const int slice = b.chunk * kWarps + wsl;
    if (role_ok && slice < p.nslices) {
      const unsigned char* base = idx_lane + static_cast<size_t>(slice) * (kSliceK / V) * IB +
                                  static_cast<size_t>(b.rbg) * item_bytes;
#pragma unroll
      for (int s = 0; s < PFB; ++s) {
        if (s < b.cnt) {
          load_idx<WORDS>(dst[s][0], base + s * item_bytes);
          load_idx<WORDS>(dst[s][1], base + s * item_bytes + row8_bytes);
        }
      }
    }
  };

  // Builds the image of `group` in slot `slot` (no barriers inside).
  auto build_image = [&](int group, int slot) {
    unsigned char* img = smem + static_cast<size_t>(slot) * img_bytes;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.cb) +
                               (static_cast<size_t>(group) * p.C << ENTRY_LOG2);
    if constexpr (V == 4 && REPL) {   // one 16-byte store = two replicas of an 8-byte entry
      const int units = p.C << (REP_LOG2 - 1);
      for (int u0 = 0; u0 < units; u0 += 4 * kThreads) {
        uint2 e[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int u = u0 + j * kThreads + tid;
          if (u < units) e[j] = __ldg(reinterpret_cast<const uint2*>(src) + (u >> (REP_LOG2 - 1)));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int u = u0 + j * kThreads + tid;
          if (u < units) reinterpret_cast<uint4*>(img)[u] = make_uint4(e[j].x, e[j].y, e[j].x, e[j].y);
        }
      }
    } else if constexpr (V == 4) {
      for (int u = tid; u < p.C; u += kThreads)
        reinterpret_cast<uint2*>(img)[u] = __ldg(reinterpret_cast<const uint2*>(src) + u);
    } else {
      const int units = p.C << REP_LOG2;
      for (int u0 = 0; u0 < units; u0 += 4 * kThreads) {
        uint4 e[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int u = u0 + j * kThreads + tid;
          if (u < units) e[j] = __ldg(reinterpret_cast<const uint4*>(src) + (u >> REP_LOG2));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int u = u0 + j * kThreads + tid;
          if (u < units) reinterpret_cast<uint4*>(img)[u] = e[j];
        }
      }
    }
  };

  // Loads the chunk's X (M rows x up to 4096 K values) with coalesced 16-byte loads and scatters every
  // piece into the staging slot of the thread(s) that own it, already in fragment-register order; then
  // each thread reads its XR registers back with 16-byte loads.  Two barriers; the staging area is
  // the same memory as the reduction buffers.
  auto load_x_fragments = [&](int chunk) {
    const int nsl = min(kWarps, p.nslices - chunk * kWarps);
    const int kc8 = nsl * (kSliceK / 8);                       // 16-byte pieces per batch row
    const __half* xbase = p.x + static_cast<size_t>(chunk) * kWarps * kSliceK;
    __syncthreads();                                           // reduction buffers are no longer read
    // rows in groups of four (four independent loads in flight per thread), pieces strided over the CTA
#pragma unroll 1
    for (int m0 = 0; m0 < p.M; m0 += 4) {
#pragma unroll 1
      for (int kg = tid; kg < kc8; kg += kThreads) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (m0 + j < p.M) v[j] = __ldg(reinterpret_cast<const uint4*>(xbase + static_cast<size_t>(m0 + j) * p.K) + kg);
        const int slice = kg >> 5, tt = (kg >> 3) & 3, i2 = kg & 7;   // owner warp slice, t4, position
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int m = m0 + j;
          if (m >= p.M) continue;
          // all row lanes of a slice need the same X
#pragma unroll 1
          for (int lr = 0; lr < p.rl; ++lr) {
            uint32_t* wbase = stage + static_cast<size_t>(lr * nsl_full + slice) * 32 * XSLOT;
            if constexpr (FORM == 1) {
              // lanes g = 2m (pairs 0, 2 of the 8-group) and g = 2m + 1 (pairs 1, 3)
              uint32_t* d0 = wbase + ((2 * m) * 4 + tt) * XSLOT + 2 * i2;
              uint32_t* d1 = wbase + ((2 * m + 1) * 4 + tt) * XSLOT + 2 * i2;
              *reinterpret_cast<uint2*>(d0) = make_uint2(v[j].x, v[j].z);
              *reinterpret_cast<uint2*>(d1) = make_uint2(v[j].y, v[j].w);
            } else if constexpr (FORM == 2) {
              // lane g = m: groups 2*i2, 2*i2+1 -> registers 4*i2 .. 4*i2+3 in order
              *reinterpret_cast<uint4*>(wbase + (m * 4 + tt) * XSLOT + 4 * i2) = v[j];
            } else {
              // lane g = m & 7, upper row selects registers +1: group i -> regs 4i+u (pair 0), 4i+2+u (pair 1)
              uint32_t* d = wbase + ((m & 7) * 4 + tt) * XSLOT + 8 * i2 + (m >> 3);
              d[0] = v[j].x; d[2] = v[j].y; d[4] = v[j].z; d[6] = v[j].w;
            }
          }
        }
      }
    }
    __syncthreads();
    const uint4* mine4 = reinterpret_cast<const uint4*>(stage + static_cast<size_t>(warp * 32 + lane) * XSLOT);
    const bool live = (FORM == 1) ? ((g >> 1) < p.M) : (g < p.M);
#pragma unroll
    for (int j = 0; j < XR / 4; ++j) {
      uint4 t = make_uint4(0, 0, 0, 0);
      if (live && role_ok && wsl < nsl) t = mine4[j];
      xf[4 * j] = t.x; xf[4 * j + 1] = t.y; xf[4 * j + 2] = t.z; xf[4 * j + 3] = t.w;
    }
    if constexpr (FORM == 3) {
      if (g + 8 >= p.M) {   // upper batch row absent: its registers were never written
#pragma unroll
        for (int i = 0; i < 16; ++i) { xf[4 * i + 1] = 0; xf[4 * i + 3] = 0; }
      }
    }
    __syncthreads();                                           // staging is free to become reduction buffers
  };

  int it = it_begin;
  Batch nb;
  {
    int chunk0 = 0, rbg0 = it;
    if (p.row_owned) rbg0 = r_begin;
    else while (rbg0 >= p.nrbg) { rbg0 -= p.nrbg; ++chunk0; }
    const int group0 = rbg0 / p.ipg;
    nb = make_batch(it, chunk0, rbg0, rbg0 - group0 * p.ipg, group0);
  }
  int parity = 0;
  bool first_batch = true;

  while (nb.cnt > 0) {
    const Batch b = nb;
    // all index loads of the batch go out first; everything up to the first lookup overlaps them
    issue_loads(b, cur);
    it += b.cnt;
    {
      int rbg = b.rbg + b.cnt, chunk = b.chunk, gpos = b.gpos + b.cnt, group = b.group;
      while (gpos >= p.ipg) { gpos -= p.ipg; ++group; }
      if (rbg >= r_end) { rbg = r_begin; group = r_begin / p.ipg; gpos = r_begin - group * p.ipg; ++chunk; }
      nb = make_batch(it, chunk, rbg, gpos, group);
    }

    const int g_first = b.group;
    const int g_last = b.group + ((b.gpos + b.cnt - 1 >= p.ipg) ? 1 : 0);   // a batch touches at most two groups
    {
      const bool need0 = (p.nslots == 1) ? (slot_group0 != g_first)
                                         : ((((g_first & 1) == 0) && slot_group0 != g_first) ||
                                            (((g_last & 1) == 0) && slot_group0 != g_last));
      const bool need1 = (p.nslots == 2) && ((((g_first & 1) == 1) && slot_group1 != g_first) ||
                                             (((g_last & 1) == 1) && slot_group1 != g_last));
      if (need0 || need1) {
        if (!first_batch) __syncthreads();   // everyone is done looking up in the old images
        if (need0) { slot_group0 = (p.nslots == 1 || (g_first & 1) == 0) ? g_first : g_last; build_image(slot_group0, 0); }
        if (need1) { slot_group1 = ((g_first & 1) == 1) ? g_first : g_last; build_image(slot_group1, 1); }
        __syncthreads();
        asm volatile("add.u32 %0, %0, 1;" : "+r"(epoch));
      }
    }

    // Everything above reads only the weights (indices, codebooks).  X, Y and the workspace belong to the
    // stream's order: when the launch was made with programmatic stream serialisation this kernel may have
    // started while its predecessor was still running, and waits here for it to complete.
    if (first_batch) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (b.chunk != loaded_chunk) {
      loaded_chunk = b.chunk;
      active = role_ok && (b.chunk * kWarps + wsl) < p.nslices;
      if constexpr (FORM == 1) {
        // B fragment of column g = (batch row g/2, pair selector g%2): for each group q of 8 K values,
        // register 0 = pair {0-1} or {2-3}, register 1 = pair {4-5} or {6-7}.  16 scattered 4-byte loads
        // per thread are cheap enough here (M <= 4) and need no barrier.
        const int m = g >> 1, h = g & 1;
        const int kt = (b.chunk * kWarps + wsl) * kSliceK + t4 * 64;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.x + static_cast<size_t>(m) * p.K + kt) + h;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint32_t v0 = 0, v1 = 0;
          if (active && m < p.M) { v0 = __ldg(src + 4 * q); v1 = __ldg(src + 4 * q + 2); }
          xf[2 * q] = v0; xf[2 * q + 1] = v1;
        }
      } else {
        load_x_fragments(b.chunk);
      }
    }
    first_batch = false;
    float* rb = red + static_cast<size_t>(parity) * (kWarps * warp_stride);
    parity ^= 1;
    float* mine = rb + warp * warp_stride;
#pragma unroll
    for (int s = 0; s < PFB; ++s) {
      if (s < b.cnt) {
        // image of this item's group
        const int grp = b.group + ((b.gpos + s >= p.ipg) ? 1 : 0);
        const uint32_t img_s = img_lane + ((p.nslots == 2 && (grp & 1)) ? img_bytes : 0u);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          float acc2[4] = {0.f, 0.f, 0.f, 0.f};  // second, independent accumulation chain
          if (active) {
            const uint32_t* w = cur[s][u].w;
            if constexpr (FORM == 1) {
              if constexpr (V == 4) {
                uint2 e[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) e[i] = lds64(img_s + (idx_at<IB>(w, i) << ENTRY_SHIFT), epoch);
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  mma_16816((q & 1) ? acc2 : acc, e[2 * q].x, e[2 * q].y, e[2 * q + 1].x, e[2 * q + 1].y, xf[2 * q], xf[2 * q + 1]);
              } else {
                uint4 e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = lds128(img_s + (idx_at<IB>(w, i) << ENTRY_SHIFT), epoch);
#pragma unroll
                for (int q = 0; q < 8; ++q) mma_16816((q & 1) ? acc2 : acc, e[q].x, e[q].y, e[q].z, e[q].w, xf[2 * q], xf[2 * q + 1]);
              }
            } else {
              constexpr int XS = (FORM == 2) ? 2 : 4;
              if constexpr (V == 4) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {   // two halves of 8 lookups keep the register count down
                  uint2 e[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) e[i] = lds64(img_s + (idx_at<IB>(w, 8 * hf + i) << ENTRY_SHIFT), epoch);
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const int ii = 8 * hf + i;
                    if constexpr (FORM == 2) mma_16816((i & 1) ? acc2 : acc, xf[XS * ii], 0u, xf[XS * ii + 1], 0u, e[i].x, e[i].y);
                    else mma_16816((i & 1) ? acc2 : acc, xf[XS * ii], xf[XS * ii + 1], xf[XS * ii + 2], xf[XS * ii + 3], e[i].x, e[i].y);
                  }
                }
              } else {
                uint4 e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = lds128(img_s + (idx_at<IB>(w, i) << ENTRY_SHIFT), epoch);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  if constexpr (FORM == 2) {
                    mma_16816(acc, xf[XS * 2 * i], 0u, xf[XS * 2 * i + 1], 0u, e[i].x, e[i].y);
                    mma_16816(acc2, xf[XS * (2 * i + 1)], 0u, xf[XS * (2 * i + 1) + 1], 0u, e[i].z, e[i].w);
                  } else {
                    mma_16816(acc, xf[XS * 2 * i], xf[XS * 2 * i + 1], xf[XS * 2 * i + 2], xf[XS * 2 * i + 3], e[i].x, e[i].y);
                    mma_16816(acc2, xf[XS * (2 * i + 1)], xf[XS * (2 * i + 1) + 1], xf[XS * (2 * i + 1) + 2],
                              xf[XS * (2 * i + 1) + 3], e[i].z, e[i].w);
                  }
                }
              }
            }
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[c] += acc2[c];
          // this warp's partial tile of the unit: [m][8 rows]
          float* dst = mine + (s * 2 + u) * unit_floats;
          if constexpr (FORM == 1) {
            if (t4 < p.M) dst[t4 * 8 + g] = acc[0] + acc[3];
          } else {
            // acc = D[batch g][rows 2t, 2t+1], D[batch g+8][rows 2t, 2t+1]
            if (g < p.M) *reinterpret_cast<float2*>(dst + g * 8 + 2 * t4) = make_float2(acc[0], acc[1]);
            if (FORM == 3 && g + 8 < p.M) *reinterpret_cast<float2*>(dst + (g + 8) * 8 + 2 * t4) = make_float2(acc[2], acc[3]);
          }
        }
      }
    }
    __syncthreads();

    // fixed-order reduction over the slices of the chunk: `lpo` lanes per output, then a butterfly.
    // Output o = ((s*rl + lr)*M + m)*16 + r; divisions by M and rl use host-made reciprocals
    // (exact for the small ranges involved).
    const int nsl = min(kWarps, p.nslices - b.chunk * kWarps);
    const int outs = b.cnt * p.rl * p.M * 16;
    const int q = tid & (p.lpo - 1);
    const int outs_per_pass = kThreads >> p.lpo_log2;
    const bool split = p.nchunks > 1 && !p.row_owned;
    const bool carry = p.nchunks > 1 && p.row_owned;   // running sums over the chunks in shared memory
    for (int o0 = 0; o0 < outs; o0 += outs_per_pass) {
      const int o = o0 + (tid >> p.lpo_log2);
      float sum = 0.f;
      int m = 0, row = 0;
      const bool valid = o < outs;
      if (valid) {
        const int r = o & 15;                 // row inside the 16-row item: unit r>>3, row r&7
        const int t = o >> 4;
        const int t1 = (t * p.inv_m) >> 16;   // t / M
        m = t - t1 * p.M;
        const int s = (t1 * p.inv_rl) >> 16;  // t1 / rl
        const int lr = t1 - s * p.rl;
        row = ((b.rbg + s) * p.rl + lr) * 16 + r;
        const float* src = rb + (lr * nsl_full) * warp_stride + (s * 2 + (r >> 3)) * unit_floats + m * 8 + (r & 7);
        for (int sl = q; sl < nsl; sl += p.lpo) sum += src[sl * warp_stride];
      }
      for (int d = p.lpo >> 1; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
      if (valid && q == 0 && carry) {
        // place of this output in the CTA's accumulator: the same for every chunk
        float* a = accbuf + (static_cast<size_t>(row >> 4) - static_cast<size_t>(r_begin) * p.rl) * (p.M * 16) + m * 16 + (row & 15);
        if (b.chunk > 0) sum += *a;
        if (b.chunk + 1 < p.nchunks) {
          *a = sum;
        } else {
          const __half h = __float2half_rn(sum);
          const size_t o_off = static_cast<size_t>(m) * p.ld_y + row;
          p.y[o_off] = h;
          for (int pq = 0; pq < p.n_peers; ++pq) p.peer_y[pq][o_off] = h;
        }
      } else if (valid && q == 0) {
        if (!split) {
          const __half h = __float2half_rn(sum);
          const size_t o_off = static_cast<size_t>(m) * p.ld_y + row;
          p.y[o_off] = h;
          for (int pq = 0; pq < p.n_peers; ++pq) p.peer_y[pq][o_off] = h;
        } else {
          __stcg(p.ws_partial + (static_cast<size_t>(b.chunk) * p.M + m) * p.N + row, sum);
        }
      }
    }
    if (split) {
      // split-K: the CTA that brings a row block's counter to nchunks sums the chunks in chunk order
      __threadfence();
      __syncthreads();
      if (tid < b.cnt) {
        const int old = atomicAdd(p.ws_counter + b.rbg + tid, 1);
        const int last = (old == p.nchunks - 1);
        if (last) p.ws_counter[b.rbg + tid] = 0;  // leave the counter zero for the next call
        s_last[tid] = last;
      }
      __syncthreads();
      __threadfence();
      for (int o = tid; o < outs; o += kThreads) {
        const int r = o & 15;
        const int t = o >> 4;
        const int t1 = (t * p.inv_m) >> 16;
        const int m = t - t1 * p.M;
        const int s = (t1 * p.inv_rl) >> 16;
        const int lr = t1 - s * p.rl;
        if (!s_last[s]) continue;
        const int row = ((b.rbg + s) * p.rl + lr) * 16 + r;
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
  }
}

// Full replication (16 or 8 copies fill a 128-byte line) when the image fits the budget, else none.
int pick_rep_log2(int v, int C, size_t budget) {
  const int rep = (v == 4) ? 4 : 3;
  return (static_cast<size_t>(C) * 2 * v << rep) <= budget ? rep : 0;
}

bool fill_params(const Problem& p, DecodeParams& d, size_t& smem_bytes) {
  if (p.M < 1 || p.M > 16) return false;
  if (!(p.v == 4 || p.v == 8)) return false;
  if (!(p.idx_bytes == 1 || (p.idx_bytes == 2 && p.v == 8))) return false;
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
  const int pfb = p.M <= 4 ? 6 : (p.M <= 8 ? (p.v == 8 ? 6 : 3) : (p.v == 8 ? 4 : 2));   // = PFB of the kernel
  d.ipg = blocks_per_group / rl;
  // lanes per output in the reduction: as many as keep all outputs of a batch in one pass
  const int outs_max = pfb * rl * p.M * 16;
  d.lpo = 1; d.lpo_log2 = 0;
  while (d.lpo * 2 <= nsl_full && d.lpo < 8 && outs_max * d.lpo * 2 <= kThreads) { d.lpo *= 2; ++d.lpo_log2; }
  d.inv_m = (65536 + p.M - 1) / p.M;
  d.inv_rl = (65536 + rl - 1) / rl;
  const size_t red_bytes = static_cast<size_t>(2) * kWarps * (pfb * 2 * p.M * 8 + 2) * sizeof(float);
  const int xr = p.M <= 4 ? 16 : (p.M <= 8 ? 32 : 64);
  const size_t stage_bytes = static_cast<size_t>(kWarps) * 32 * (xr + 4) * sizeof(uint32_t);
  const size_t work_bytes = red_bytes > stage_bytes ? red_bytes : stage_bytes;
  d.rep_log2 = pick_rep_log2(p.v, p.C, 64 * 1024);
  const size_t img_bytes = static_cast<size_t>(p.C) * entry << d.rep_log2;
  // a second resident image lets batches straddle a group boundary without a rebuild in between
  d.nslots = (!single && 2 * img_bytes + work_bytes <= 210 * 1024) ? 2 : 1;
  smem_bytes = d.nslots * img_bytes + work_bytes;
  if (smem_bytes > 220 * 1024) return false;
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

namespace {
int device_sms() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}
// Row-owned walk of the K chunks (see DecodeParams::row_owned): worth it when there are several chunks and
// enough row blocks that an even split of them over the SMs is balanced (at least six per CTA: measured 20 %
// faster at 12 per CTA and K = 8192, but 12 % slower at 3.5 per CTA and K = 28672), and when the running sums of
// a CTA's rows fit shared memory next to everything else.
bool plan_row_owned(DecodeParams& d, size_t& smem, int M) {
  if (d.nchunks <= 1) return false;
  const int sms = device_sms();
  if (d.nrbg < 6 * sms) return false;
  const int per_cta = (d.nrbg + sms - 1) / sms;
  const size_t acc_bytes = static_cast<size_t>(per_cta) * d.rl * M * 16 * sizeof(float);
  const size_t off = (smem + 15) & ~static_cast<size_t>(15);
  if (off + acc_bytes > 220 * 1024) return false;
  d.row_owned = 1;
  d.acc_offset = static_cast<int>(off);
  smem = off + acc_bytes;
  return true;
}
}  // namespace

int launch_decode(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s) {
  DecodeParams d{};
  size_t smem;
  if (!fill_params(p, d, smem)) return VQG_ERR_UNSUPPORTED;
  const bool row_owned = plan_row_owned(d, smem, p.M);
  if (d.nchunks > 1 && !row_owned) {
    const size_t need = decode_workspace_bytes(p);
    if (ws == nullptr || ws_bytes < need) return VQG_ERR_WORKSPACE;
    if (static_cast<size_t>(d.nrbg) * sizeof(int) > kCounterBytes) return VQG_ERR_UNSUPPORTED;
    d.ws_counter = static_cast<int*>(ws);
    d.ws_partial = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + kCounterBytes);
  }
  d.status = device_status_ptr();

  const int sms = device_sms();
  // what is dealt out over the CTAs: (chunk, row block) items, or row blocks in the row-owned mode
  const long long items = row_owned ? d.nrbg : static_cast<long long>(d.nchunks) * d.nrbg;
  const int grid = static_cast<int>(items < sms ? items : sms);
  d.items_q = static_cast<int>(items / grid);
  d.items_r = static_cast<int>(items % grid);

  const int form = p.M <= 4 ? 1 : (p.M <= 8 ? 2 : 3);
  using KernelT = void (*)(const DecodeParams);
  KernelT k = nullptr;
#define VQG_PICK(V_, IB_)                                                                                \
  if (p.v == V_ && p.idx_bytes == IB_) {                                                                 \
    if (d.rep_log2 > 0)                                                                                  \
      k = form == 1 ? vq_decode_kernel<V_, IB_, 1, true>                                                 \
                    : (form == 2 ? vq_decode_kernel<V_, IB_, 2, true> : vq_decode_kernel<V_, IB_, 3, true>); \
    else                                                                                                 \
      k = form == 1 ? vq_decode_kernel<V_, IB_, 1, false>                                                \
                    : (form == 2 ? vq_decode_kernel<V_, IB_, 2, false> : vq_decode_kernel<V_, IB_, 3, false>); \
  }
  VQG_PICK(4, 1) VQG_PICK(8, 1) VQG_PICK(8, 2)
#undef VQG_PICK
  if (!k) return VQG_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return VQG_ERR_LAUNCH;
  // Programmatic dependent launch: set-up, the codebook image and the first batch of index loads of this
  // launch overlap the tail of the kernel before it in the stream (see the wait inside the kernel).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, k, d);
  count_launch();
  return cuda_status(e == cudaSuccess ? cudaGetLastError() : e);
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
  d.items_q = static_cast<int>(items / grid);
  d.items_r = static_cast<int>(items % grid);
  const int form = p.M <= 4 ? 1 : (p.M <= 8 ? 2 : 3);
  using KernelT = void (*)(const DecodeParams);
  KernelT k = nullptr;
#define VQG_PICK(V_, IB_)                                                                                \
  if (p.v == V_ && p.idx_bytes == IB_) {                                                                 \
    if (d.rep_log2 > 0)                                                                                  \
      k = form == 1 ? vq_decode_kernel<V_, IB_, 1, true>                                                 \
                    : (form == 2 ? vq_decode_kernel<V_, IB_, 2, true> : vq_decode_kernel<V_, IB_, 3, true>); \
    else                                                                                                 \
      k = form == 1 ? vq_decode_kernel<V_, IB_, 1, false>                                                \
                    : (form == 2 ? vq_decode_kernel<V_, IB_, 2, false> : vq_decode_kernel<V_, IB_, 3, false>); \
  }
  VQG_PICK(4, 1) VQG_PICK(8, 1) VQG_PICK(8, 2)
#undef VQG_PICK
  if (!k) return VQG_ERR_UNSUPPORTED;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return VQG_ERR_LAUNCH;
  k<<<grid, kThreads, smem, s>>>(d);
  count_launch();
  return cuda_status(cudaGetLastError());
}

}  // namespace vqg
