/*
 * vqg.h -- C ABI of the B200 (sm_100a) vector-quantised GEMM library, libvqg_b200.so.
 *
 * Plain C: device pointers, sizes and an opaque stream handle; no torch or pybind types.
 * Every entry point returns a status code (VQG_OK == 0) and never throws, prints or
 * falls back to a CPU path.  All pointers are DEVICE pointers unless stated otherwise.
 *
 * Two weight formats are understood (``layout``):
 *
 *   VQG_LAYOUT_BL   W[n, v*j + r] = codebook[n / rows_per_codebook][ idx[n, j] ][r]
 *                   idx [N, K/v] (uint8 or uint16), codebook [G, C, v] fp16,
 *                   Y[M, N] = X[M, K] * W^T            (the benchmark configurations)
 *
 *   VQG_LAYOUT_REF  Wdec[k, 2*n + r] = codebook[n / 4][ w[k, n] ][r]
 *                   w [K, Nq] uint8, codebook [Nq/4, 256, 2] fp16,
 *                   Y[M, 2*Nq] = X[M, K] * Wdec        (the reference's own format,
 *                   reference bench.py:37-57 and strategy_1/src.cu:268-321)
 *
 * X and Y are fp16 row-major; accumulation is fp32; Y is rounded once to fp16.
 */
#ifndef VQG_H_
#define VQG_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define VQG_API __attribute__((visibility("default")))
#else
#define VQG_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
enum {
  VQG_OK = 0,
  VQG_ERR_BAD_ARG = 1,        /* null pointer, non-positive size, misaligned pointer            */
  VQG_ERR_UNSUPPORTED = 2,    /* a (v, C, index width, layout, path) combination not built      */
  VQG_ERR_WORKSPACE = 3,      /* workspace missing or smaller than vqg_workspace_bytes()        */
  VQG_ERR_LAUNCH = 4,         /* the CUDA runtime or driver refused a call                      */
  VQG_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait ran out (see vqg_device_status)     */
  VQG_ERR_NO_DEVICE = 6,      /* no usable sm_100 device / driver                                */
  VQG_ERR_TOO_LARGE = 7,      /* problem needs more scratch than the built-in static buffer has */
  VQG_ERR_NO_MEMORY = 8       /* the device had no memory left to load this library's code and data */
};

enum { VQG_LAYOUT_BL = 0, VQG_LAYOUT_REF = 1 };

/* idx_bytes value for 12-bit indices packed two to three bytes (bytes [a & 255, (a >> 8) | ((b & 15) << 4),
 * b >> 4] for the pair a, b -- what vqg_pack12 writes).  1.5 bits per weight at v = 8 instead of the 2 bits
 * of uint16 storage.  No counterpart in the reference (uint8 indices only). */
#define VQG_IDX_PACKED12 12

/* kernel selection for vqg_gemm_path(); VQG_PATH_AUTO is what vqg_gemm() uses */
enum {
  VQG_PATH_AUTO = 0,
  VQG_PATH_GENERIC = 1,  /* shape-agnostic CUDA-core kernel                                     */
  VQG_PATH_DECODE = 2,   /* M <= 16: TMA index tiles + codebook lookups + mma.sync, split-K      */
  VQG_PATH_TENSOR = 3,   /* tcgen05 / TMEM / TMA warp-specialised kernel, fused dequant, 1 CTA  */
  VQG_PATH_TWO_PHASE = 4,/* dequantise to workspace, then the dense tcgen05 kernel              */
  VQG_PATH_TENSOR_PAIR = 5, /* the fused kernel on CTA pairs (tcgen05 cta_group::2, 256x256 tiles) */
  VQG_PATH_TENSOR_TS = 6,  /* CTA pairs, dequantised weights as the MMA's tensor-memory operand;
                              with a workspace the K loops are dealt out evenly over the pairs    */
  VQG_PATH_SMALL_TS = 7    /* M <= 128: tensor-memory operand, K loop split evenly over the SMs    */
};

/* Library version (major*10000 + minor*100 + patch). */
VQG_API int vqg_version(void);

/* Static string for a status code.  (No reference counterpart: the reference checks no errors;
 * strategy_3/naive/src.cu:42-54 prints cudaGetLastError and continues.) */
VQG_API const char* vqg_status_string(int status);

/* Bytes of scratch the given problem needs (0 if none).  In every workspace the first
 * vqg_workspace_counter_bytes() bytes hold arrival counters and must be zero when the
 * workspace is first used (cudaMemset once after allocation); the library leaves them zero and
 * puts every other payload behind them, so one buffer can serve any sequence of calls that
 * do not overlap on the GPU.
 * Replaces the per-call temporaries of the reference (strategy_1/src.cu:351 allocates
 * a [K, 2*Nq] matrix on every call). */
VQG_API size_t vqg_workspace_bytes(int M, int N, int K, int v, int C, int idx_bytes,
                           int rows_per_codebook, int layout, int path);
VQG_API size_t vqg_workspace_counter_bytes(void);

/* The kernel (VQG_PATH_*) that VQG_PATH_AUTO resolves to for a problem with 1024-byte aligned operands
 * and ld_y = N.  Routing is by measurement on B200: decode kernel up to 8 batch rows, and up to 16 when
 * K <= 4096 and the codebook has at most 256 entries; small-batch tensor-memory kernel up to 96;
 * CTA-pair kernel above. */
VQG_API int vqg_auto_path(int M, int N, int K, int v, int C, int idx_bytes, int rows_per_codebook, int layout);

/* Y = X * dequant(idx, codebook)^T.  Replaces `torch::Tensor e2e_gemm(input, w, codebook)`
 * (reference bind.cpp:3,7; host launchers strategy_2/bsz128/src.cu:255-316 and siblings).
 *   N                  output columns (BL: rows of idx; REF: 2*Nq)
 *   v, C               sub-vector length and codebook entries (REF: v=2, C=256)
 *   idx_bytes          1 (uint8), 2 (uint16), or VQG_IDX_PACKED12 (vqg_gemm, vqg_gemm_path, vqg_dequant,
 *                      vqg_workspace_bytes, vqg_auto_path only; BL layout): two 12-bit indices in three
 *                      bytes as vqg_pack12 writes them, K/v even, C <= 4096; a row of the index matrix
 *                      is K/v * 3/2 bytes
 *   (every index must be below C.  A larger one is the caller's error; the kernels keep it from addressing
 *   past the codebook -- 16-bit and packed indices are clamped to the last entry, 8-bit ones stay inside the
 *   256-entry image region -- so the result for that weight is meaningless but the launch completes)
 *   rows_per_codebook  BL: output rows sharing a codebook, 0 = one codebook for the matrix
 *                      REF: ignored (8 output columns per codebook)
 *   stream             cudaStream_t (NULL = legacy default stream, as the reference uses)
 * Ordering: X, Y and the workspace follow the stream's order.  The WEIGHTS (idx, codebook) are
 * taken to be constant: for M <= 128 the kernels are launched with programmatic stream
 * serialisation and read indices and codebooks while the kernel ahead of them on the stream may
 * still be finishing (they wait for it before touching X, Y or the workspace).  Weights written by
 * this library's own entry points (vqg_quantize_*, vqg_pack12 / vqg_unpack12) are taken care of: the
 * first product enqueued on that stream afterwards is launched in plain stream order.  If another
 * KERNEL of the caller's has just written the weights on the same stream, put a synchronisation
 * (event, host wait) between it and this call; copies (cudaMemcpyAsync) need nothing. */
VQG_API int vqg_gemm(const void* x, const void* idx, const void* codebook, void* y,
             int M, int N, int K, int v, int C, int idx_bytes, int rows_per_codebook,
             int layout, void* workspace, size_t workspace_bytes, void* stream);

/* Same, with the kernel chosen by the caller (tests and benchmarks). */
VQG_API int vqg_gemm_path(const void* x, const void* idx, const void* codebook, void* y,
                  int M, int N, int K, int v, int C, int idx_bytes, int rows_per_codebook,
                  int layout, int path, void* workspace, size_t workspace_bytes, void* stream);

/* Dequantised weights, bit-exact gather.  BL: w_out [N, K]; REF: w_out [K, N] (N = 2*Nq).
 * Replaces `dequant_kernel` of the reference's two-phase variant (strategy_1/src.cu:268-321). */
VQG_API int vqg_dequant(const void* idx, const void* codebook, void* w_out,
                int N, int K, int v, int C, int idx_bytes, int rows_per_codebook,
                int layout, void* stream);

/* Dense fp16 GEMM with fp32 accumulation.  Replaces `torch::Tensor gemm(input, w)`
 * (reference bind.cpp:4,8; ref_gemm/cublas_gemm_fp16.cu:15-48).
 *   w_is_kn = 1: w is [K, N] row-major (the reference's convention);  0: w is [N, K]. */
VQG_API int vqg_dense_gemm(const void* x, const void* w, void* y, int M, int N, int K, int w_is_kn,
                   void* workspace, size_t workspace_bytes, void* stream);
VQG_API size_t vqg_dense_workspace_bytes(int M, int N, int K, int w_is_kn);

/* N-sharded multi-GPU mode (no reference counterpart: the reference is single-GPU, device 0
 * is hard-coded at strategy_1/src.cu:343).  This rank owns output columns
 * [rank*N_local, (rank+1)*N_local) of a Y with ld_y = nranks*N_local columns; idx/codebook are
 * the rank's shard.  y_peers[r] (HOST array of nranks DEVICE pointers) is the base of the full
 * Y buffer on rank r (peer-mapped); the kernel epilogue stores the rank's column block into
 * every one of them.  y_peers[rank] must be local.  With nranks == 1 this is vqg_gemm with a
 * leading dimension. */
VQG_API int vqg_gemm_sharded(const void* x, const void* idx, const void* codebook,
                     void* const* y_peers, int rank, int nranks,
                     int M, int N_local, int K, int v, int C, int idx_bytes, int rows_per_codebook,
                     void* workspace, size_t workspace_bytes, void* stream);

/* The same product with the gather done by the NVLink switch: y_multicast is the multicast (NVLS) address of
 * the ranks' Y buffers -- a mapping through which one store lands in every rank's buffer at the same offset,
 * this rank's included (cuMulticast* objects; torch's symmetric memory exposes it as `multicast_ptr`).  For
 * shapes that run the prefill kernel the epilogue then issues ONE 16-byte multimem store per 16 bytes of
 * output instead of one store per rank: a rank's block leaves over NVLink once and the switch replicates it.
 * Other shapes, y_multicast == NULL and nranks == 1 behave exactly like vqg_gemm_sharded.  No reference
 * counterpart.  Every rank of the multicast group must stay alive while the mapping is bound. */
VQG_API int vqg_gemm_sharded_mc(const void* x, const void* idx, const void* codebook,
                        void* const* y_peers, void* y_multicast, int rank, int nranks,
                        int M, int N_local, int K, int v, int C, int idx_bytes, int rows_per_codebook,
                        void* workspace, size_t workspace_bytes, void* stream);

/* The same product for a SLAB of this rank's columns: output columns [col0, col0 + N_cols) of a Y with ld_y
 * columns on every rank (col0 and ld_y multiples of 8); idx / codebook are the shard of exactly those columns.
 * For callers that hand a rank's block over in pieces (their consumer starts on the first columns while the rest
 * is computed).  Launches of one step share the workspace and follow one another in stream order.  As a way
 * to start the NVLink stream earlier (a small first slab) it did not pay: on 2 GPUs a 512-column first launch
 * made the C5-shaped step 15 % slower.  vqg_gemm_sharded_mc is this call with col0 = rank * N_local, ld_y = nranks *
 * N_local.  No reference counterpart. */
VQG_API int vqg_gemm_sharded_cols(const void* x, const void* idx, const void* codebook,
                          void* const* y_peers, void* y_multicast, int rank, int nranks,
                          int M, int N_cols, int K, int v, int C, int idx_bytes, int rows_per_codebook,
                          long long col0, long long ld_y,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Barrier across the ranks of a sharded product, to be enqueued after vqg_gemm_sharded* (or
 * vqg_gemm_rowparallel) on the same stream: when it completes on a rank, every rank's stores into this rank's
 * buffers have landed.  flag_ptrs[r] (HOST array of nranks DEVICE pointers) is rank r's flag array: nranks
 * 32-bit words in peer-mapped memory, zero when first used, never reset; flag_ptrs[rank] is local.  `epoch`
 * is the number of this barrier: 1 for the first, one more for each following barrier on these flags, the
 * same on every rank.  The wait is bounded: if a rank has not arrived after limit_cycles SM cycles
 * (1e3 .. 2e10) the kernel records code 11 in the device status word and returns -- vqg_device_status() then
 * reports VQG_ERR_DEVICE_TIMEOUT and the device stays usable.  Plain system-scope stores and loads over
 * NVLink; no multicast.  No reference counterpart (the reference is single-GPU, strategy_1/src.cu:343). */
VQG_API int vqg_rank_barrier(void* const* flag_ptrs, int rank, int nranks, unsigned epoch,
                     long long limit_cycles, void* stream);

/* Small-batch product (M <= 16) for callers that must not allocate device memory.  (This entry
 * point has no counterpart in the reference.)
 *
 * Who needs it: host programs that hand the whole of the GPU's memory to their own pool when
 * they start (inference servers commonly do), so that a cudaMalloc made later from inside a
 * plugin fails or eats into memory the host believes it owns; and callers on a latency-critical
 * path, because cudaMalloc and cudaFree synchronise the whole device.  vqg_gemm() needs a
 * caller-allocated workspace when K > 4096 (split-K partial sums); this variant of the same
 * kernel keeps that scratch in a fixed array of VQG_NOALLOC_SCRATCH_BYTES inside the library
 * image instead -- every GPU that loads the library holds those bytes until the process exits.
 * The call itself makes no cudaMalloc / cudaFree and calls no allocating library routine.
 *
 * Limits and rules:
 *   - same shapes as the decode path of vqg_gemm (BL layout, M <= 16, K > 0, K % 256 == 0,
 *     N % 8 == 0, whole 16-row tiles per codebook); anything else returns VQG_ERR_UNSUPPORTED --
 *     there is no other kernel behind this entry (K == 0 writes zeros, as vqg_gemm does);
 *   - the scratch a problem needs is what vqg_workspace_bytes(..., VQG_PATH_DECODE) reports: nothing
 *     up to K = 4096 and for large matrices, whose CTAs keep their rows' running sums on chip;
 *     64 KiB + ceil(K/4096) * M * N * 4 bytes for K > 4096 on matrices with few rows.  Beyond
 *     VQG_NOALLOC_SCRATCH_BYTES the call returns VQG_ERR_TOO_LARGE;
 *   - the first call on each device looks up the device address of the array (the device must be
 *     current).  With CUDA's lazy module loading that lookup is also the moment the runtime puts
 *     this library's code and the array itself onto the device, so it needs those few MiB to be
 *     free: make the first call on every device BEFORE the host hands the rest of the memory to
 *     its pool, and before any stream capture on that device.  If the memory is already gone the
 *     call returns VQG_ERR_NO_MEMORY.  Later calls leave the amount of free memory unchanged;
 *   - all calls on a device share the one array and it keeps the previous call's contents (the
 *     call re-zeroes the counters it needs on `stream`): two calls that overlap on the GPU -- on
 *     different streams, or from different threads -- race.  Serialise them. */
#define VQG_NOALLOC_SCRATCH_BYTES (4u << 20)
VQG_API int vqg_gemm_small_batch_noalloc(const void* x, const void* idx, const void* codebook, void* y,
                                 int M, int N, int K, int v, int C, int idx_bytes,
                                 int rows_per_codebook, void* stream);

/* ---- Row-parallel (K-sharded) product with reduce-scatter (no counterpart in the reference) ----
 * The second half of a tensor-parallel MLP: rank r holds K_local = K/G input features -- x_local
 * [M, K_local] (what the N-sharded first half left on this rank) and idx_local [N, K_local/v] (its
 * K slice of every weight row) -- and all codebooks.  Every rank computes a partial [M, N]; the
 * output columns are cut into G blocks of N/G (a multiple of 128) and rank o owns block o.
 *
 * vqg_gemm_rowparallel: writes this rank's partial of block o, fp16 [M, N/G], to part_of_owner[o]
 *   for every o (host array of G device pointers; part_of_owner[rank] is local memory, the others
 *   are peer-mapped).  By convention part_of_owner[o] is slot `rank` of owner o's buffer
 *   [G][M][N/G].  For M > 128 the prefill kernel stores each finished tile straight to its owner
 *   with a TMA tensor store (no multicast); other shapes compute into scratch and scatter.
 * After a barrier across the ranks (all partials have landed):
 * vqg_reduce_slots: y_local[M, cols] = sum over the G slots of part_local [G][M][cols], fp32
 *   accumulation in slot order (deterministic), one rounding to fp16.
 * Workspace: vqg_rowparallel_workspace_bytes(), 1024-byte aligned, zeroed once, one per stream. */
VQG_API size_t vqg_rowparallel_workspace_bytes(int M, int N, int K_local, int v, int C, int idx_bytes,
                                               int rows_per_codebook);
VQG_API int vqg_gemm_rowparallel(const void* x_local, const void* idx_local, const void* codebook,
                                 void* const* part_of_owner, int nranks, int M, int N, int K_local, int v,
                                 int C, int idx_bytes, int rows_per_codebook, void* workspace,
                                 size_t workspace_bytes, void* stream);
VQG_API int vqg_reduce_slots(const void* part_local, void* y_local, int nranks, int M, int cols,
                             long long ld_y, void* stream);

/* ---- Gated product: the step after the path in a gated MLP (no counterpart in the reference) ----
 * The weight matrix holds (gate, up) row pairs: row 2i is gate row i and row 2i+1 is up row i
 * (BL layout, idx [2*N_out, K/v], one codebook per `rows_per_codebook` of those interleaved rows).
 *     Y[m, i] = SiLU(X[m,:] . g_i) * (X[m,:] . u_i),   SiLU(t) = t / (1 + exp(-t)),
 * both dot products accumulated in fp32 and combined in fp32 before the single rounding to fp16.
 * Y is [M, N_out] row-major.  For M > 128 and shapes the prefill kernel takes, the combination
 * happens in that kernel's epilogue and the two products never reach memory; otherwise the product
 * is written to scratch inside the workspace and combined by a second kernel.  Workspace of
 * vqg_swiglu_workspace_bytes() bytes, 1024-byte aligned, zeroed once, one per stream. */
VQG_API size_t vqg_swiglu_workspace_bytes(int M, int N_out, int K, int v, int C, int idx_bytes, int rows_per_codebook);
VQG_API int vqg_gemm_swiglu(const void* x, const void* idx, const void* codebook, void* y, int M, int N_out, int K,
                            int v, int C, int idx_bytes, int rows_per_codebook, void* workspace,
                            size_t workspace_bytes, void* stream);

/* ---- Residual (multi-codebook) weights ---------------------------------------------------------
 * The reference only hints at this format: `#define RESIDUAL 1` (strategy_1/src.cu:18) is defined and never
 * used.  Here: n_stages index matrices idx [S][N][K/v] and codebook sets codebook [S][G][C][v], each stage
 * laid out like the BL format and stored one after the other; the weight is the running fp16 sum of the
 * stages' entries,
 *     W_0 = codebook_0[g(n)][idx_0[n,j]],   W_s = fp16(W_{s-1} + codebook_s[g(n)][idx_s[n,j]])   (round to nearest even),
 * so S stages of b bits give S*b bits per sub-vector.  vqg_dequant_residual writes exactly that W [N, K].
 * vqg_gemm_residual computes Y = X * W^T: for M > 16 and two stages the prefill kernel holds both stages'
 * codebook images and adds the two entries (HADD2) on their way into tensor memory -- the tensor core sees
 * W bit for bit; for M <= 16 the decode kernel walks the stages like further chunks of K (the products of
 * the stages are summed in fp32, which differs from the product with the rounded W by less than the fp16
 * rounding of W); other shapes dequantise into the workspace and run the dense kernel, or use the generic
 * kernel.  n_stages == 1 is the plain product.  Workspace: vqg_residual_workspace_bytes(), 1024-byte
 * aligned, zeroed once. */
VQG_API size_t vqg_residual_workspace_bytes(int M, int N, int K, int v, int C, int idx_bytes, int rows_per_codebook,
                                            int n_stages);
VQG_API int vqg_gemm_residual(const void* x, const void* idx, const void* codebook, void* y, int M, int N, int K,
                              int v, int C, int idx_bytes, int rows_per_codebook, int n_stages, void* workspace,
                              size_t workspace_bytes, void* stream);
VQG_API int vqg_dequant_residual(const void* idx, const void* codebook, void* w_out, int N, int K, int v, int C,
                                 int idx_bytes, int rows_per_codebook, int n_stages, void* stream);

/* ---- Quantiser: the step before the product ------------------------------------------------
 * The reference has no quantiser (bench.py:83-85 fills `w` with random bytes); these entry points
 * turn a dense fp16 weight W[N, K] into the BL format on the GPU.  All pointers are device
 * pointers; W must be 16-byte aligned; v in {2, 4, 8}; C <= 256 with 1-byte indices, any C whose
 * fp32 copy (C*v*4 bytes) fits 200 KiB of shared memory with 2-byte indices.
 *
 * vqg_quantize_assign: idx[n, j] = the entry of codebook g(n) nearest to W[n, jv : jv+v], where
 *   distance = sum over i ascending of (float(w_i) - float(c_i))^2 with every subtraction,
 *   multiplication and addition rounded to fp32 separately (no fused multiply-add), and the
 *   lowest index wins among equal distances -- a rule a CPU restates bit for bit.
 * vqg_quantize_update: one k-means (Lloyd) update -- every codebook entry becomes the mean of
 *   the sub-vectors whose index names it (entries nobody chose keep their value).  Sums are exact
 *   64-bit fixed-point (fp16 values are multiples of 2^-24), hence independent of the order of
 *   accumulation; mean = (float)((double)sum * 2^-24 / count), rounded to fp16.  `workspace` of
 *   vqg_quantize_workspace_bytes() bytes, 16-byte aligned; the call zeroes it itself.
 * vqg_pack12 / vqg_unpack12: `values` (even) 12-bit indices held in uint16 <-> 3 bytes per pair:
 *   bytes [a & 255, (a >> 8) | ((b & 15) << 4), b >> 4]; the uint16 side must be 4-byte aligned. */
VQG_API int vqg_quantize_assign(const void* w, const void* codebook, void* idx_out, int N, int K, int v, int C,
                                int idx_bytes, int rows_per_codebook, void* stream);
VQG_API size_t vqg_quantize_workspace_bytes(int N, int v, int C, int rows_per_codebook);
VQG_API int vqg_quantize_update(const void* w, const void* idx, void* codebook_inout, void* workspace,
                                size_t workspace_bytes, int N, int K, int v, int C, int idx_bytes,
                                int rows_per_codebook, void* stream);
VQG_API int vqg_pack12(const void* idx_u16, void* packed_out, long long values, void* stream);
VQG_API int vqg_unpack12(const void* packed, void* idx_u16_out, long long values, void* stream);

/* Failure-path self-test (no counterpart in the reference, whose kernels wait without bound,
 * e.g. the cuda::barrier waits of strategy_3/wasp/src.cu:262-319): launches one small kernel that
 * waits on an mbarrier nobody signals, with the same bounded-wait routine the pipelined kernels use
 * and a limit of `limit_cycles` SM cycles (1e3 .. 2e9, i.e. at most about a second).  The kernel
 * records code 10 in the status word and returns normally; vqg_device_status() then reports
 * VQG_ERR_DEVICE_TIMEOUT with that code, and the device stays usable. */
VQG_API int vqg_selftest_bounded_wait(long long limit_cycles, void* stream);

/* Reads and clears the device-side status word of the current device: 0 if no bounded wait has
 * run out since the last call, else a code naming the wait.  Synchronises the device. */
VQG_API int vqg_device_status(int* code_out);

/* Number of kernels this library has launched in the calling process (all streams). */
VQG_API unsigned long long vqg_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* VQG_H_ */
