// extern "C" surface of libvqg_b200.so: argument checks, kernel selection, workspace rules.
// Declarations and the reference interfaces they replace are in include/vqg.h.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace vqg {

namespace {
std::atomic<unsigned long long> g_launches{0};
std::mutex g_mu;
int* g_status[64] = {};
// The status word kernels report a run-out wait in: a zero-initialised device variable of the library image
// (every device that loads the library has its own copy), so that no call ever allocates device memory.
__device__ int g_status_word[64];
}  // namespace

void count_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

namespace {
std::mutex g_dirty_mu;
cudaStream_t g_dirty[16];
int g_ndirty = 0;
}  // namespace

void note_weights_written(cudaStream_t s) {
  std::lock_guard<std::mutex> lk(g_dirty_mu);
  for (int i = 0; i < g_ndirty; ++i)
    if (g_dirty[i] == s) return;
  if (g_ndirty < 16) g_dirty[g_ndirty++] = s;
  else g_dirty[0] = s;   // table full: streams may then be reported late; the documented contract still holds
}

bool take_weights_written(cudaStream_t s) {
  std::lock_guard<std::mutex> lk(g_dirty_mu);
  for (int i = 0; i < g_ndirty; ++i)
    if (g_dirty[i] == s) {
      g_dirty[i] = g_dirty[--g_ndirty];
      return true;
    }
  return false;
}

cudaError_t ensure_status_word() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev]) return cudaSuccess;
  void* p = nullptr;
  e = cudaGetSymbolAddress(&p, g_status_word);
  if (e != cudaSuccess) return e;
  g_status[dev] = static_cast<int*>(p);
  return cudaSuccess;
}

int* device_status_ptr() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < 64) ? g_status[dev] : nullptr;
}

namespace {

bool aligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

// `packed_ok`: the entry point also takes VQG_IDX_PACKED12 (two 12-bit indices in three bytes); only the plain
// product and the dequantisation do.
int check_common(const void* x, const void* idx, const void* cb, const void* y, int M, int N, int K, int v, int C,
                 int idx_bytes, int layout, bool packed_ok = false) {
  if (M < 0 || N < 0 || K < 0) return VQG_ERR_BAD_ARG;
  if (layout != VQG_LAYOUT_BL && layout != VQG_LAYOUT_REF) return VQG_ERR_BAD_ARG;
  if (M == 0 || N == 0) return VQG_OK;
  if (!y || !aligned(y, 2)) return VQG_ERR_BAD_ARG;
  if (K > 0 && (!x || !idx || !cb || !aligned(x, 2) || !aligned(cb, 2))) return VQG_ERR_BAD_ARG;
  if (layout == VQG_LAYOUT_REF) {
    if (v != 2 || C != 256 || idx_bytes != 1) return VQG_ERR_UNSUPPORTED;
    if (N % 8 != 0) return VQG_ERR_BAD_ARG;  // 4 index columns (8 outputs) per codebook
  } else {
    if (v < 1 || C < 1) return VQG_ERR_BAD_ARG;
    if (idx_bytes == VQG_IDX_PACKED12) {
      if (!packed_ok) return VQG_ERR_UNSUPPORTED;
      if (K % v != 0 || (K / v) % 2 != 0 || C > 4096) return VQG_ERR_BAD_ARG;   // pairs never straddle rows
      return VQG_OK;
    }
    if (idx_bytes != 1 && idx_bytes != 2) return VQG_ERR_UNSUPPORTED;
    if (K % v != 0) return VQG_ERR_BAD_ARG;
    if (idx_bytes == 1 && C > 256) return VQG_ERR_BAD_ARG;
    if (C > 65536) return VQG_ERR_BAD_ARG;
    if (idx_bytes == 2 && !aligned(idx, 2)) return VQG_ERR_BAD_ARG;
  }
  return VQG_OK;
}

Problem make_problem(const void* x, const void* idx, const void* cb, void* y, int M, int N, int K, int v, int C,
                     int idx_bytes, int rows_per_cb, long long ld_y) {
  Problem p{};
  p.x = static_cast<const __half*>(x);
  p.idx = idx;
  p.cb = static_cast<const __half*>(cb);
  p.y = static_cast<__half*>(y);
  p.M = M; p.N = N; p.K = K; p.v = v; p.C = C; p.idx_bytes = idx_bytes;
  p.rows_per_cb = (rows_per_cb <= 0 || rows_per_cb > N) ? (N > 0 ? N : 1) : rows_per_cb;
  p.ld_y = ld_y;
  p.n_peers = 0;
  return p;
}

int auto_path(const Problem& p, int layout) {
  if (layout == VQG_LAYOUT_REF) {
    return dense_supported(p.M, p.N, p.K) && p.M >= 32 ? VQG_PATH_TWO_PHASE : VQG_PATH_GENERIC;
  }
  if (p.K == 0) return VQG_PATH_GENERIC;
  if (p.idx_bytes == VQG_IDX_PACKED12) {
    // packed indices: the small-batch tensor-memory kernel unpacks them itself; larger batches dequantise first
    if (p.M <= 128 && small_ts_supported(p)) return VQG_PATH_SMALL_TS;
    if (dense_supported(p.M, p.N, p.K) && (p.v == 2 || p.v == 4 || p.v == 8) && aligned(p.cb, static_cast<size_t>(2 * p.v)))
      return VQG_PATH_TWO_PHASE;
    return VQG_PATH_GENERIC;
  }
  // Measured routing (B200, CUDA-graph replay over index buffers larger than L2).  Register-level decode kernel:
  // fastest up to 8 batch rows on every matrix tried (4 MB ... 29 MB of indices, 256- and 4096-entry codebooks), and
  // up to 16 rows while K fits one chunk of its warps (K <= 4096) and the codebook its replicated image (C4 weights,
  // M = 16: 16.9 us against 20.3 us); with more chunks or an unreplicated codebook its 16-row form loses (70B
  // weights, M = 16: 54 us against 41 us).  The small-batch tensor-memory kernel takes over from there up to 96
  // rows; above that the pair kernel with its 256-row batch tile is as fast or faster even half empty.
  const bool small_ok = small_ts_supported(p);
  if (p.M <= 16 && decode_supported(p)) {
    const bool prefer_small = small_ok && p.M > 8 && (p.K > 4096 || p.C > 256);
    if (!prefer_small) return VQG_PATH_DECODE;
  }
  if (p.M <= 96 && small_ok) return VQG_PATH_SMALL_TS;
  if (p.M > 96 && tensor_ts_supported(p)) return VQG_PATH_TENSOR_TS;
  if (p.M <= 128 && small_ok) return VQG_PATH_SMALL_TS;
  if (p.M > 128 && tensor_pair_supported(p)) return VQG_PATH_TENSOR_PAIR;
  if (p.M > 16 && tensor_supported(p)) return VQG_PATH_TENSOR;
  // the dequantising kernels read whole codebook entries: a codebook that is not aligned to its entry size
  // (2v bytes) goes to the generic kernel, which reads it half by half
  if (p.M > 16 && dense_supported(p.M, p.N, p.K) && (p.v == 2 || p.v == 4 || p.v == 8) &&
      aligned(p.cb, static_cast<size_t>(2 * p.v)))
    return VQG_PATH_TWO_PHASE;
  return VQG_PATH_GENERIC;
}

// Every workspace starts with the counter region (kept zero by the split-K kernel); payloads of all
// paths live behind it so that one cached buffer can serve any sequence of calls.
size_t two_phase_bytes(int N, int K) { return kCounterBytes + static_cast<size_t>(N) * K * 2; }

int run(const Problem& p, int layout, int path, void* ws, size_t ws_bytes, cudaStream_t s) {
  if (p.M == 0 || p.N == 0) return VQG_OK;
  if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
  if (path == VQG_PATH_AUTO) path = auto_path(p, layout);
  switch (path) {
    case VQG_PATH_GENERIC:
      return launch_generic(p, layout, s);
    case VQG_PATH_DECODE:
      if (layout != VQG_LAYOUT_BL) return VQG_ERR_UNSUPPORTED;
      return launch_decode(p, ws, ws_bytes, s);
    case VQG_PATH_TENSOR:
      if (layout != VQG_LAYOUT_BL) return VQG_ERR_UNSUPPORTED;
      return launch_tensor(p, s);
    case VQG_PATH_TENSOR_PAIR:
      if (layout != VQG_LAYOUT_BL) return VQG_ERR_UNSUPPORTED;
      return launch_tensor_pair(p, s);
    case VQG_PATH_TENSOR_TS:
      if (layout != VQG_LAYOUT_BL) return VQG_ERR_UNSUPPORTED;
      return launch_tensor_ts(p, ws, ws_bytes, s);
    case VQG_PATH_SMALL_TS:
      if (layout != VQG_LAYOUT_BL) return VQG_ERR_UNSUPPORTED;
      return launch_small_ts(p, ws, ws_bytes, s);
    case VQG_PATH_TWO_PHASE: {
      if (!dense_supported(p.M, p.N, p.K)) return VQG_ERR_UNSUPPORTED;
      const size_t need = two_phase_bytes(p.N, p.K);
      if (!ws || ws_bytes < need || !aligned(ws, 1024)) return VQG_ERR_WORKSPACE;
      __half* w = reinterpret_cast<__half*>(static_cast<unsigned char*>(ws) + kCounterBytes);
      int st;
      if (layout == VQG_LAYOUT_BL)
        st = launch_dequant_bl(p.idx, p.cb, w, p.N, p.K, p.v, p.C, p.idx_bytes, p.rows_per_cb, s);
      else
        st = launch_dequant_ref(static_cast<const uint8_t*>(p.idx), p.cb, w, p.N / 2, p.K, /*transposed=*/true, s);
      if (st != VQG_OK) return st;
      if (p.M > 128) return launch_dense_pair(p.x, w, p.y, p.M, p.N, p.K, p.ld_y, p.n_peers, p.peer_y, s);
      return launch_dense(p.x, w, p.y, p.M, p.N, p.K, p.ld_y, p.n_peers, p.peer_y, s);
    }
    default:
      return VQG_ERR_BAD_ARG;
  }
}

}  // namespace
}  // namespace vqg

using namespace vqg;

extern "C" {

int vqg_version(void) { return 100; }

const char* vqg_status_string(int status) {
  switch (status) {
    case VQG_OK: return "ok";
    case VQG_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, negative size, K not a multiple of v)";
    case VQG_ERR_UNSUPPORTED: return "unsupported combination of v, C, index width, layout or path";
    case VQG_ERR_WORKSPACE: return "workspace missing, misaligned or smaller than vqg_workspace_bytes()";
    case VQG_ERR_LAUNCH: return "CUDA runtime or driver call failed";
    case VQG_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case VQG_ERR_NO_DEVICE: return "no usable CUDA device";
    case VQG_ERR_TOO_LARGE: return "problem needs more scratch than the library's built-in static buffer holds";
    case VQG_ERR_NO_MEMORY: return "out of device memory while loading the library's code and static data onto the device";
    default: return "unknown status";
  }
}

int vqg_auto_path(int M, int N, int K, int v, int C, int idx_bytes, int rows_per_codebook, int layout) {
  if (M <= 0 || N <= 0 || K < 0) return VQG_PATH_GENERIC;
  void* dummy = reinterpret_cast<void*>(static_cast<uintptr_t>(1024));
  Problem p = make_problem(dummy, dummy, dummy, dummy, M, N, K, v, C, idx_bytes, rows_per_codebook, N);
  return auto_path(p, layout);
}

size_t vqg_workspace_counter_bytes(void) { return kCounterBytes; }

size_t vqg_workspace_bytes(int M, int N, int K, int v, int C, int idx_bytes, int rows_per_codebook, int layout,
                           int path) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // pointers only matter for alignment checks; use aligned dummies
  void* dummy = reinterpret_cast<void*>(static_cast<uintptr_t>(1024));
  Problem p = make_problem(dummy, dummy, dummy, dummy, M, N, K, v, C, idx_bytes, rows_per_codebook, N);
  if (path == VQG_PATH_AUTO) path = auto_path(p, layout);
  if (path == VQG_PATH_DECODE) return decode_workspace_bytes(p);
  if (path == VQG_PATH_SMALL_TS) return small_ts_workspace_bytes(p);
  if (path == VQG_PATH_TENSOR_TS) return tensor_ts_workspace_bytes(p);
  if (path == VQG_PATH_TWO_PHASE) return two_phase_bytes(N, K);
  return 0;
}

int vqg_gemm_path(const void* x, const void* idx, const void* codebook, void* y, int M, int N, int K, int v, int C,
                  int idx_bytes, int rows_per_codebook, int layout, int path, void* workspace,
                  size_t workspace_bytes, void* stream) {
  const int st = check_common(x, idx, codebook, y, M, N, K, v, C, idx_bytes, layout, /*packed_ok=*/true);
  if (st != VQG_OK) return st;
  Problem p = make_problem(x, idx, codebook, y, M, N, K, v, C, idx_bytes, rows_per_codebook, N);
  return run(p, layout, path, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int vqg_gemm(const void* x, const void* idx, const void* codebook, void* y, int M, int N, int K, int v, int C,
             int idx_bytes, int rows_per_codebook, int layout, void* workspace, size_t workspace_bytes, void* stream) {
  return vqg_gemm_path(x, idx, codebook, y, M, N, K, v, C, idx_bytes, rows_per_codebook, layout, VQG_PATH_AUTO,
                       workspace, workspace_bytes, stream);
}

int vqg_dequant(const void* idx, const void* codebook, void* w_out, int N, int K, int v, int C, int idx_bytes,
                int rows_per_codebook, int layout, void* stream) {
  if (N < 0 || K < 0) return VQG_ERR_BAD_ARG;
  if (N == 0 || K == 0) return VQG_OK;
  if (!idx || !codebook || !w_out) return VQG_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (layout == VQG_LAYOUT_REF) {
    if (v != 2 || C != 256 || idx_bytes != 1 || N % 8 != 0) return VQG_ERR_UNSUPPORTED;
    return launch_dequant_ref(static_cast<const uint8_t*>(idx), static_cast<const __half*>(codebook),
                              static_cast<__half*>(w_out), N / 2, K, false, s);
  }
  if (layout != VQG_LAYOUT_BL) return VQG_ERR_BAD_ARG;
  if (v < 1 || C < 1 || K % v != 0) return VQG_ERR_BAD_ARG;
  if (idx_bytes == VQG_IDX_PACKED12) {
    if ((K / v) % 2 != 0 || C > 4096) return VQG_ERR_BAD_ARG;
  } else {
    if (idx_bytes != 1 && idx_bytes != 2) return VQG_ERR_UNSUPPORTED;
    if (idx_bytes == 1 && C > 256) return VQG_ERR_BAD_ARG;
  }
  if (!aligned(w_out, 16) || !aligned(codebook, 16) ||
      !aligned(idx, idx_bytes == VQG_IDX_PACKED12 ? 1 : static_cast<size_t>(idx_bytes)))
    return VQG_ERR_BAD_ARG;
  const int rpc = (rows_per_codebook <= 0 || rows_per_codebook > N) ? N : rows_per_codebook;
  return launch_dequant_bl(idx, static_cast<const __half*>(codebook), static_cast<__half*>(w_out), N, K, v, C,
                           idx_bytes, rpc, s);
}

size_t vqg_dense_workspace_bytes(int M, int N, int K, int w_is_kn) {
  (void)M;
  return w_is_kn ? kCounterBytes + static_cast<size_t>(N) * K * 2 : 0;
}

int vqg_dense_gemm(const void* x, const void* w, void* y, int M, int N, int K, int w_is_kn, void* workspace,
                   size_t workspace_bytes, void* stream) {
  if (M < 0 || N < 0 || K < 0) return VQG_ERR_BAD_ARG;
  if (M == 0 || N == 0) return VQG_OK;
  if (!x || !w || !y) return VQG_ERR_BAD_ARG;
  if (!dense_supported(M, N, K)) return VQG_ERR_UNSUPPORTED;
  if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* w_nk = static_cast<const __half*>(w);
  if (w_is_kn) {
    if (!workspace || workspace_bytes < vqg_dense_workspace_bytes(M, N, K, 1) || !aligned(workspace, 1024))
      return VQG_ERR_WORKSPACE;
    __half* wt = reinterpret_cast<__half*>(static_cast<unsigned char*>(workspace) + kCounterBytes);
    const int st = launch_transpose(static_cast<const __half*>(w), wt, K, N, s);
    if (st != VQG_OK) return st;
    w_nk = wt;
  }
  if (M > 128) return launch_dense_pair(static_cast<const __half*>(x), w_nk, static_cast<__half*>(y), M, N, K, N, 0, nullptr, s);
  return launch_dense(static_cast<const __half*>(x), w_nk, static_cast<__half*>(y), M, N, K, N, 0, nullptr, s);
}

int vqg_gemm_sharded(const void* x, const void* idx, const void* codebook, void* const* y_peers, int rank,
                     int nranks, int M, int N_local, int K, int v, int C, int idx_bytes, int rows_per_codebook,
                     void* workspace, size_t workspace_bytes, void* stream) {
  return vqg_gemm_sharded_mc(x, idx, codebook, y_peers, nullptr, rank, nranks, M, N_local, K, v, C, idx_bytes,
                             rows_per_codebook, workspace, workspace_bytes, stream);
}

int vqg_rank_barrier(void* const* flag_ptrs, int rank, int nranks, unsigned epoch, long long limit_cycles, void* stream) {
  if (nranks < 1 || nranks > 8 || rank < 0 || rank >= nranks || !flag_ptrs) return VQG_ERR_BAD_ARG;
  if (limit_cycles < 1000 || limit_cycles > 20000000000LL) return VQG_ERR_BAD_ARG;   // at most about ten seconds
  unsigned* f[8] = {};
  for (int r = 0; r < nranks; ++r) {
    if (!flag_ptrs[r] || !aligned(flag_ptrs[r], 4)) return VQG_ERR_BAD_ARG;
    f[r] = static_cast<unsigned*>(flag_ptrs[r]);
  }
  if (nranks == 1) return VQG_OK;
  if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
  return launch_rank_barrier(f, rank, nranks, epoch, limit_cycles, static_cast<cudaStream_t>(stream));
}

int vqg_gemm_sharded_cols(const void* x, const void* idx, const void* codebook, void* const* y_peers, void* y_multicast,
                          int rank, int nranks, int M, int N_cols, int K, int v, int C, int idx_bytes,
                          int rows_per_codebook, long long col0, long long ld_y, void* workspace, size_t workspace_bytes,
                          void* stream) {
  if (nranks < 1 || nranks > 8 || rank < 0 || rank >= nranks || !y_peers) return VQG_ERR_BAD_ARG;
  if (col0 < 0 || N_cols < 0 || ld_y < col0 + N_cols || col0 % 8 != 0 || ld_y % 8 != 0) return VQG_ERR_BAD_ARG;
  if (y_multicast && !aligned(y_multicast, 16)) return VQG_ERR_BAD_ARG;
  for (int r = 0; r < nranks; ++r)
    if (!y_peers[r]) return VQG_ERR_BAD_ARG;
  void* y_local = static_cast<__half*>(y_peers[rank]) + col0;
  const int st = check_common(x, idx, codebook, y_local, M, N_cols, K, v, C, idx_bytes, VQG_LAYOUT_BL);
  if (st != VQG_OK) return st;
  Problem p = make_problem(x, idx, codebook, y_local, M, N_cols, K, v, C, idx_bytes, rows_per_codebook, ld_y);
  for (int r = 0; r < nranks; ++r)
    if (r != rank) p.peer_y[p.n_peers++] = static_cast<__half*>(y_peers[r]) + col0;
  // through the switch only where the kernel that will run has the multimem epilogue (the prefill kernel);
  // every other kernel keeps its per-rank stores
  if (y_multicast && nranks > 1 && auto_path(p, VQG_LAYOUT_BL) == VQG_PATH_TENSOR_TS)
    p.mc_y = static_cast<__half*>(y_multicast) + col0;
  return run(p, VQG_LAYOUT_BL, VQG_PATH_AUTO, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int vqg_gemm_sharded_mc(const void* x, const void* idx, const void* codebook, void* const* y_peers, void* y_multicast,
                        int rank, int nranks, int M, int N_local, int K, int v, int C, int idx_bytes,
                        int rows_per_codebook, void* workspace, size_t workspace_bytes, void* stream) {
  if (nranks < 1 || nranks > 8 || rank < 0 || rank >= nranks || N_local < 0) return VQG_ERR_BAD_ARG;
  return vqg_gemm_sharded_cols(x, idx, codebook, y_peers, y_multicast, rank, nranks, M, N_local, K, v, C, idx_bytes,
                               rows_per_codebook, static_cast<long long>(rank) * N_local,
                               static_cast<long long>(nranks) * N_local, workspace, workspace_bytes, stream);
}

namespace {
size_t align_up(size_t n, size_t a) { return (n + a - 1) / a * a; }
// Scratch for the two products sits behind whatever the product itself needs, and never inside the counter
// region at the head of a workspace (a cached workspace serves other calls that expect those counters zero).
size_t swiglu_scratch_offset(size_t inner) { return align_up(inner < vqg::kCounterBytes ? vqg::kCounterBytes : inner, 1024); }
// fused epilogue when the prefill kernel takes the shape, otherwise product into scratch + elementwise kernel
bool swiglu_fused(const vqg::Problem& p) { return p.M > 128 && vqg::tensor_ts_supported(p); }
}  // namespace

size_t vqg_swiglu_workspace_bytes(int M, int N_out, int K, int v, int C, int idx_bytes, int rows_per_codebook) {
  if (M <= 0 || N_out <= 0 || K <= 0 || N_out > 0x3fffffff) return 0;
  void* dummy = reinterpret_cast<void*>(static_cast<uintptr_t>(1024));
  const int N = 2 * N_out;
  Problem p = make_problem(dummy, dummy, dummy, dummy, M, N, K, v, C, idx_bytes, rows_per_codebook, N_out);
  if (swiglu_fused(p)) return tensor_ts_workspace_bytes(p);
  const size_t inner = vqg_workspace_bytes(M, N, K, v, C, idx_bytes, rows_per_codebook, VQG_LAYOUT_BL, VQG_PATH_AUTO);
  return swiglu_scratch_offset(inner) + static_cast<size_t>(M) * N * 2;
}

int vqg_gemm_swiglu(const void* x, const void* idx, const void* codebook, void* y, int M, int N_out, int K, int v, int C,
                    int idx_bytes, int rows_per_codebook, void* workspace, size_t workspace_bytes, void* stream) {
  if (N_out < 0 || N_out > 0x3fffffff) return VQG_ERR_BAD_ARG;
  const int N = 2 * N_out;
  const int st = check_common(x, idx, codebook, y, M, N, K, v, C, idx_bytes, VQG_LAYOUT_BL);
  if (st != VQG_OK) return st;
  if (M == 0 || N == 0) return VQG_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Problem p = make_problem(x, idx, codebook, y, M, N, K, v, C, idx_bytes, rows_per_codebook, N_out);
  if (swiglu_fused(p)) {
    if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
    return launch_tensor_ts(p, workspace, workspace_bytes, s, /*gated=*/true);
  }
  const size_t need = vqg_workspace_bytes(M, N, K, v, C, idx_bytes, rows_per_codebook, VQG_LAYOUT_BL, VQG_PATH_AUTO);
  const size_t inner = swiglu_scratch_offset(need);
  if (!workspace || workspace_bytes < inner + static_cast<size_t>(M) * N * 2 || !aligned(workspace, 1024)) return VQG_ERR_WORKSPACE;
  __half* tmp = reinterpret_cast<__half*>(static_cast<unsigned char*>(workspace) + inner);
  Problem q = make_problem(x, idx, codebook, tmp, M, N, K, v, C, idx_bytes, rows_per_codebook, N);
  const int st2 = run(q, VQG_LAYOUT_BL, VQG_PATH_AUTO, need ? workspace : nullptr, need, s);
  if (st2 != VQG_OK) return st2;
  return launch_swiglu(tmp, static_cast<__half*>(y), M, N_out, N_out, s);
}

size_t vqg_rowparallel_workspace_bytes(int M, int N, int K_local, int v, int C, int idx_bytes, int rows_per_codebook) {
  if (M <= 0 || N <= 0 || K_local <= 0) return 0;
  void* dummy = reinterpret_cast<void*>(static_cast<uintptr_t>(1024));
  Problem p = make_problem(dummy, dummy, dummy, dummy, M, N, K_local, v, C, idx_bytes, rows_per_codebook, N);
  if (p.M > 128 && tensor_ts_supported(p)) return tensor_ts_workspace_bytes(p);
  const size_t inner = vqg_workspace_bytes(M, N, K_local, v, C, idx_bytes, rows_per_codebook, VQG_LAYOUT_BL, VQG_PATH_AUTO);
  return swiglu_scratch_offset(inner) + static_cast<size_t>(M) * N * 2;
}

int vqg_gemm_rowparallel(const void* x_local, const void* idx_local, const void* codebook, void* const* part_of_owner,
                         int nranks, int M, int N, int K_local, int v, int C, int idx_bytes, int rows_per_codebook,
                         void* workspace, size_t workspace_bytes, void* stream) {
  if (nranks < 1 || nranks > 8 || !part_of_owner || N < 0 || (N > 0 && N % (nranks * 128) != 0)) return VQG_ERR_BAD_ARG;
  for (int o = 0; o < nranks; ++o)
    if (!part_of_owner[o] || !aligned(part_of_owner[o], 16)) return VQG_ERR_BAD_ARG;
  const int st = check_common(x_local, idx_local, codebook, part_of_owner[0], M, N, K_local, v, C, idx_bytes, VQG_LAYOUT_BL);
  if (st != VQG_OK) return st;
  if (M == 0 || N == 0) return VQG_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int cols = N / nranks;
  Problem p = make_problem(x_local, idx_local, codebook, part_of_owner[0], M, N, K_local, v, C, idx_bytes, rows_per_codebook, N);
  if (p.M > 128 && tensor_ts_supported(p)) {
    p.n_owners = nranks;
    p.owner_cols = cols;
    for (int o = 0; o < nranks; ++o) p.owner_part[o] = static_cast<__half*>(part_of_owner[o]);
    if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
    return launch_tensor_ts(p, workspace, workspace_bytes, s, /*gated=*/false);
  }
  // other shapes: the product into scratch, then one kernel that hands every owner its block
  const size_t need = vqg_workspace_bytes(M, N, K_local, v, C, idx_bytes, rows_per_codebook, VQG_LAYOUT_BL, VQG_PATH_AUTO);
  const size_t inner = swiglu_scratch_offset(need);
  if (!workspace || workspace_bytes < inner + static_cast<size_t>(M) * N * 2 || !aligned(workspace, 1024)) return VQG_ERR_WORKSPACE;
  __half* tmp = reinterpret_cast<__half*>(static_cast<unsigned char*>(workspace) + inner);
  Problem q = make_problem(x_local, idx_local, codebook, tmp, M, N, K_local, v, C, idx_bytes, rows_per_codebook, N);
  const int st2 = run(q, VQG_LAYOUT_BL, VQG_PATH_AUTO, need ? workspace : nullptr, need, s);
  if (st2 != VQG_OK) return st2;
  __half* owners[8];
  for (int o = 0; o < nranks; ++o) owners[o] = static_cast<__half*>(part_of_owner[o]);
  return launch_scatter_blocks(tmp, owners, nranks, M, cols, s);
}

int vqg_reduce_slots(const void* part_local, void* y_local, int nranks, int M, int cols, long long ld_y, void* stream) {
  if (!part_local || !y_local) return (M == 0 || cols == 0) ? VQG_OK : VQG_ERR_BAD_ARG;
  return launch_reduce_slots(static_cast<const __half*>(part_local), static_cast<__half*>(y_local), nranks, M, cols, ld_y,
                             static_cast<cudaStream_t>(stream));
}

int vqg_gemm_small_batch_noalloc(const void* x, const void* idx, const void* codebook, void* y, int M, int N, int K,
                                 int v, int C, int idx_bytes, int rows_per_codebook, void* stream) {
  const int st = check_common(x, idx, codebook, y, M, N, K, v, C, idx_bytes, VQG_LAYOUT_BL);
  if (st != VQG_OK) return st;
  if (M == 0 || N == 0) return VQG_OK;
  if (M > 16) return VQG_ERR_UNSUPPORTED;
  Problem p = make_problem(x, idx, codebook, y, M, N, K, v, C, idx_bytes, rows_per_codebook, N);
  if (K == 0) return launch_generic(p, VQG_LAYOUT_BL, static_cast<cudaStream_t>(stream));   // Y = 0, as vqg_gemm gives
  return launch_decode_static(p, static_cast<cudaStream_t>(stream));
}

// ---- residual (multi-codebook) weights -------------------------------------------------------------
namespace {
// which kernel serves a residual problem: 2 decode, 6 prefill (two resident images), 4 dequantise + dense, 1 generic
int residual_route(const vqg::Problem& p) {
  if (p.K == 0) return VQG_PATH_GENERIC;
  if (p.M <= 16 && vqg::decode_supported(p)) return VQG_PATH_DECODE;
  const int groups = (p.N + p.rows_per_cb - 1) / p.rows_per_cb;
  if (p.n_stages == 2 && p.M > 16 && vqg::tensor_ts_supported(p) &&
      (static_cast<size_t>(groups) * p.C * p.v * 2) % 16 == 0)
    return VQG_PATH_TENSOR_TS;
  if (vqg::dense_supported(p.M, p.N, p.K) && (p.v == 2 || p.v == 4 || p.v == 8)) return VQG_PATH_TWO_PHASE;
  return VQG_PATH_GENERIC;
}
}  // namespace

size_t vqg_residual_workspace_bytes(int M, int N, int K, int v, int C, int idx_bytes, int rows_per_codebook, int n_stages) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (n_stages <= 1) return vqg_workspace_bytes(M, N, K, v, C, idx_bytes, rows_per_codebook, VQG_LAYOUT_BL, VQG_PATH_AUTO);
  void* dummy = reinterpret_cast<void*>(static_cast<uintptr_t>(1024));
  Problem p = make_problem(dummy, dummy, dummy, dummy, M, N, K, v, C, idx_bytes, rows_per_codebook, N);
  p.n_stages = n_stages;
  switch (residual_route(p)) {
    case VQG_PATH_DECODE: return decode_workspace_bytes(p);
    case VQG_PATH_TENSOR_TS: return tensor_ts_workspace_bytes(p);
    case VQG_PATH_TWO_PHASE: return two_phase_bytes(N, K);
    default: return 0;
  }
}

int vqg_gemm_residual(const void* x, const void* idx, const void* codebook, void* y, int M, int N, int K, int v, int C,
                      int idx_bytes, int rows_per_codebook, int n_stages, void* workspace, size_t workspace_bytes,
                      void* stream) {
  if (n_stages < 1 || n_stages > 8) return VQG_ERR_BAD_ARG;
  if (n_stages == 1)
    return vqg_gemm(x, idx, codebook, y, M, N, K, v, C, idx_bytes, rows_per_codebook, VQG_LAYOUT_BL, workspace,
                    workspace_bytes, stream);
  const int st = check_common(x, idx, codebook, y, M, N, K, v, C, idx_bytes, VQG_LAYOUT_BL);
  if (st != VQG_OK) return st;
  if (M == 0 || N == 0) return VQG_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Problem p = make_problem(x, idx, codebook, y, M, N, K, v, C, idx_bytes, rows_per_codebook, N);
  p.n_stages = n_stages;
  if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
  switch (residual_route(p)) {
    case VQG_PATH_DECODE:
      return launch_decode(p, workspace, workspace_bytes, s);
    case VQG_PATH_TENSOR_TS:
      return launch_tensor_ts(p, workspace, workspace_bytes, s);
    case VQG_PATH_TWO_PHASE: {
      const size_t need = two_phase_bytes(N, K);
      if (!workspace || workspace_bytes < need || !aligned(workspace, 1024)) return VQG_ERR_WORKSPACE;
      __half* w = reinterpret_cast<__half*>(static_cast<unsigned char*>(workspace) + kCounterBytes);
      const int st2 = launch_dequant_bl_residual(idx, p.cb, w, N, K, v, C, idx_bytes, p.rows_per_cb, n_stages, s);
      if (st2 != VQG_OK) return st2;
      if (M > 128) return launch_dense_pair(p.x, w, p.y, M, N, K, N, 0, nullptr, s);
      return launch_dense(p.x, w, p.y, M, N, K, N, 0, nullptr, s);
    }
    default:
      return launch_generic(p, VQG_LAYOUT_BL, s);
  }
}

int vqg_dequant_residual(const void* idx, const void* codebook, void* w_out, int N, int K, int v, int C, int idx_bytes,
                         int rows_per_codebook, int n_stages, void* stream) {
  if (N < 0 || K < 0 || n_stages < 1 || n_stages > 8) return VQG_ERR_BAD_ARG;
  if (N == 0 || K == 0) return VQG_OK;
  if (!idx || !codebook || !w_out) return VQG_ERR_BAD_ARG;
  if (v < 1 || C < 1 || K % v != 0) return VQG_ERR_BAD_ARG;
  if (idx_bytes != 1 && idx_bytes != 2) return VQG_ERR_UNSUPPORTED;
  if (idx_bytes == 1 && C > 256) return VQG_ERR_BAD_ARG;
  const int rpc = (rows_per_codebook <= 0 || rows_per_codebook > N) ? N : rows_per_codebook;
  return launch_dequant_bl_residual(idx, static_cast<const __half*>(codebook), static_cast<__half*>(w_out), N, K, v, C,
                                    idx_bytes, rpc, n_stages, static_cast<cudaStream_t>(stream));
}

int vqg_quantize_assign(const void* w, const void* codebook, void* idx_out, int N, int K, int v, int C, int idx_bytes,
                        int rows_per_codebook, void* stream) {
  if (!w || !codebook || !idx_out || N < 0 || K < 0) return VQG_ERR_BAD_ARG;
  if (N == 0 || K == 0) return VQG_OK;
  return launch_quantize_assign(static_cast<const __half*>(w), static_cast<const __half*>(codebook), idx_out, N, K, v, C,
                                idx_bytes, rows_per_codebook, static_cast<cudaStream_t>(stream));
}

size_t vqg_quantize_workspace_bytes(int N, int v, int C, int rows_per_codebook) {
  if (N <= 0 || v <= 0 || C <= 0) return 0;
  return quantize_workspace_bytes(N, v, C, rows_per_codebook);
}

int vqg_quantize_update(const void* w, const void* idx, void* codebook_inout, void* workspace, size_t workspace_bytes,
                        int N, int K, int v, int C, int idx_bytes, int rows_per_codebook, void* stream) {
  if (!w || !idx || !codebook_inout || N < 0 || K < 0) return VQG_ERR_BAD_ARG;
  if (N == 0 || K == 0) return VQG_OK;
  return launch_quantize_update(static_cast<const __half*>(w), idx, static_cast<__half*>(codebook_inout), workspace,
                                workspace_bytes, N, K, v, C, idx_bytes, rows_per_codebook,
                                static_cast<cudaStream_t>(stream));
}

int vqg_pack12(const void* idx_u16, void* packed_out, long long values, void* stream) {
  if (values < 0 || (values > 0 && (!idx_u16 || !packed_out))) return VQG_ERR_BAD_ARG;
  return launch_pack12(idx_u16, packed_out, values, true, static_cast<cudaStream_t>(stream));
}

int vqg_unpack12(const void* packed, void* idx_u16_out, long long values, void* stream) {
  if (values < 0 || (values > 0 && (!packed || !idx_u16_out))) return VQG_ERR_BAD_ARG;
  return launch_pack12(packed, idx_u16_out, values, false, static_cast<cudaStream_t>(stream));
}

int vqg_selftest_bounded_wait(long long limit_cycles, void* stream) {
  if (ensure_status_word() != cudaSuccess) return VQG_ERR_NO_DEVICE;
  return launch_selftest_wait(limit_cycles, static_cast<cudaStream_t>(stream));
}

int vqg_device_status(int* code_out) {
  if (!code_out) return VQG_ERR_BAD_ARG;
  *code_out = 0;
  int* p = device_status_ptr();
  if (!p) return VQG_OK;  // nothing has run on this device yet
  if (cudaDeviceSynchronize() != cudaSuccess) return VQG_ERR_LAUNCH;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return VQG_ERR_LAUNCH;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  *code_out = v;
  return v == 0 ? VQG_OK : VQG_ERR_DEVICE_TIMEOUT;
}

unsigned long long vqg_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
