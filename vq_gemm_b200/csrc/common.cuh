// Shared declarations of the sm_100a VQ-GEMM kernels: problem descriptor, launcher
// prototypes, the device status word and small PTX helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/vqg.h"

namespace vqg {

// One VQ-GEMM problem, BL layout (see include/vqg.h).  ld_y lets the output live inside a
// wider matrix (column shard of a gathered Y).
struct Problem {
  const __half* x;      // [M, K]
  const void* idx;      // [N, K/v] uint8 or uint16
  const __half* cb;     // [G, C, v]
  __half* y;            // [M, ld_y], columns [0, N) written
  int M, N, K;
  int v, C, idx_bytes;
  int rows_per_cb;      // >= 1; N when one codebook serves the matrix
  long long ld_y;
  // multi-GPU epilogue: additional copies of the output block (peer-mapped), may be 0
  int n_peers;
  __half* peer_y[8];
  // multi-GPU epilogue through the switch: the multicast address of the output block (NVLS mapping of the ranks'
  // symmetric Y buffers); one multimem store then lands in every rank's copy, this rank's included, and y /
  // peer_y are not written.  Null = off.  Only the prefill kernel (weights through tensor memory) uses it.
  __half* mc_y;
  // row-parallel (K-sharded) mode: the output columns are cut into n_owners blocks of owner_cols columns and
  // block o is written, as this rank's partial sum, to owner_part[o] ([M, owner_cols] fp16, possibly peer
  // memory) instead of y.  0 = off.
  int n_owners;
  int owner_cols;
  __half* owner_part[8];
  // residual (multi-codebook) weights: n_stages index matrices [S][N][K/v] and codebook sets [S][G][C][v], one
  // after the other in memory; W = the running fp16 sum over the stages of the looked-up entries.  0 or 1 = plain.
  int n_stages;
};

// Device status word: 0 = fine; otherwise the code of the first bounded wait that ran out.
enum DeviceStatus : int {
  DS_OK = 0,
  DS_TMA_FULL_TIMEOUT = 1,   // consumer waited for a TMA-filled stage
  DS_STAGE_EMPTY_TIMEOUT = 2,// producer waited for a free stage
  DS_B_READY_TIMEOUT = 3,    // MMA warp waited for dequantised B
  DS_ACC_FULL_TIMEOUT = 4,   // epilogue waited for the accumulator
  DS_ACC_EMPTY_TIMEOUT = 5,  // MMA warp waited for the epilogue to drain TMEM
  DS_SPLITK_TIMEOUT = 6,
  DS_DEQUANT_SYNC_TIMEOUT = 7,
  DS_PEER_READY_TIMEOUT = 8, // pair leader waited for the second CTA's operands
  DS_EPILOGUE_SYNC_TIMEOUT = 9,
  DS_SELFTEST_TIMEOUT = 10,  // the self-test kernel's wait on a barrier nobody signals
  DS_RANK_BARRIER_TIMEOUT = 11,  // the cross-GPU barrier waited for a rank that did not arrive
};
int* device_status_ptr();          // device address of the status word of the current device
cudaError_t ensure_status_word();  // looks its address up on first use (per device); allocates nothing

void count_launch(int n = 1);

// Weights written by this library on a stream (the quantiser, the index packer): the small-batch kernels read
// indices and codebooks BEFORE they wait for the kernel ahead of them when launched with programmatic stream
// serialisation, so the first product enqueued on that stream afterwards is launched without that attribute
// (ordinary stream order).  note_weights_written marks the stream; take_weights_written reports and clears it.
void note_weights_written(cudaStream_t s);
bool take_weights_written(cudaStream_t s);

// ---- launchers (each returns a VQG_* status) -------------------------------------------
int launch_dequant_bl(const void* idx, const __half* cb, __half* w, int N, int K, int v, int C,
                      int idx_bytes, int rows_per_cb, cudaStream_t s);
int launch_dequant_ref(const uint8_t* w, const __half* cb, __half* out, int Nq, int K, bool transposed,
                       cudaStream_t s);
// residual weights: w[n, k] = fp16 running sum over `stages` of codebook_s[g(n)][idx_s[n, k/v]][k%v]
int launch_dequant_bl_residual(const void* idx, const __half* cb, __half* w, int N, int K, int v, int C, int idx_bytes,
                               int rows_per_cb, int stages, cudaStream_t s);
int launch_generic(const Problem& p, int layout, cudaStream_t s);

bool decode_supported(const Problem& p);
size_t decode_workspace_bytes(const Problem& p);
int launch_decode(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s);
int launch_decode_static(const Problem& p, cudaStream_t s);  // scratch in a static device array

bool tensor_supported(const Problem& p);
int launch_tensor(const Problem& p, cudaStream_t s);
bool dense_supported(int M, int N, int K);
// Y[M,N] = X[M,K] * W[N,K]^T, all fp16, fp32 accumulate (tcgen05).
int launch_dense(const __half* x, const __half* w_nk, __half* y, int M, int N, int K, long long ld_y,
                 int n_peers, __half* const* peer_y, cudaStream_t s);
bool tensor_pair_supported(const Problem& p);
int launch_tensor_pair(const Problem& p, cudaStream_t s);   // CTA-pair (cta_group::2) version
int launch_dense_pair(const __half* x, const __half* w_nk, __half* y, int M, int N, int K, long long ld_y,
                      int n_peers, __half* const* peer_y, cudaStream_t s);
bool tensor_ts_supported(const Problem& p);
size_t tensor_ts_workspace_bytes(const Problem& p);
// gated: weight rows are (gate, up) pairs and Y[M, N/2] = SiLU(X g) * (X u)
int launch_tensor_ts(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s, bool gated = false);
// elementwise SiLU(g) * u over interleaved columns: in [M, 2*n_out] -> out [M, n_out] (leading dimension ld_out)
// y[M, cols] (leading dimension ld_y) = sum over s < slots of part[s][M][cols] (fp16 in, fp32 sum in slot order)
int launch_reduce_slots(const __half* part, __half* y, int slots, int M, int cols, long long ld_y, cudaStream_t s);
// tmp[M, n_owners*cols] -> owner_part[o][M, cols] for every o (plain stores, possibly to peer memory)
int launch_scatter_blocks(const __half* tmp, __half* const* owner_part, int n_owners, int M, int cols, cudaStream_t s);
int launch_swiglu(const __half* in, __half* out, int M, int n_out, long long ld_out, cudaStream_t s);     // weights through tensor memory (A operand)
bool small_ts_supported(const Problem& p);
size_t small_ts_workspace_bytes(const Problem& p);
int launch_small_ts(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t s);   // M <= 128, stream-K
// quantiser (the step before the product): nearest-entry search, exact k-means update, 12-bit packing
size_t quantize_workspace_bytes(int N, int v, int C, int rows_per_cb);
int launch_quantize_assign(const __half* w, const __half* cb, void* idx, int N, int K, int v, int C, int idx_bytes,
                           int rows_per_cb, cudaStream_t s);
int launch_quantize_update(const __half* w, const void* idx, __half* cb, void* ws, size_t ws_bytes, int N, int K, int v,
                           int C, int idx_bytes, int rows_per_cb, cudaStream_t s);
int launch_pack12(const void* in, void* out, long long values, bool pack, cudaStream_t s);
int launch_selftest_wait(long long limit_cycles, cudaStream_t s);   // see vqg_selftest_bounded_wait
// cross-GPU barrier on epoch flags in peer-mapped memory, bounded wait (see vqg_rank_barrier)
int launch_rank_barrier(unsigned* const* flags, int rank, int nranks, unsigned epoch, long long limit_cycles, cudaStream_t s);
int launch_transpose(const __half* in, __half* out, int rows, int cols, cudaStream_t s);

constexpr size_t kCounterBytes = 64 * 1024;  // arrival counters at the head of a workspace

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? VQG_OK : VQG_ERR_LAUNCH; }

// ---- device helpers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

}  // namespace vqg
