/* C ABI of the B200 (sm_100a) GEMM library: FP16/BF16 GEMM with fp32
 * accumulation, FP8 e4m3 blockwise-quantised GEMM with the output's 1x128
 * re-quantisation fused in, and the blockwise quantisers that prepare its
 * operands.
 *
 * Every entry point is the C form of a host launcher of the reference project
 * (file:line given per function, paths relative to the reference root) and
 * keeps its conventions:
 *   - all pointers are device pointers owned by the caller; nothing is
 *     allocated, C is fully overwritten;
 *   - the work is enqueued on `stream` and the call returns without
 *     synchronising;
 *   - matrices are dense row-major with no padding.
 * Where the reference launchers throw std::runtime_error, these return a
 * status code; the C++ wrappers under llmmm_b200/src/mm re-throw it.
 *
 * There is no CPU path: on a machine without an sm_100 GPU every compute
 * entry point returns LLMMM_ERR_UNSUPPORTED.
 */
#ifndef LLMMM_C_H
#define LLMMM_C_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without requiring the CUDA headers. */
typedef struct CUstream_st* llmmm_stream_t;

enum {
  LLMMM_OK              = 0,
  LLMMM_ERR_SHAPE       = 1, /* shape / alignment not supported ("M or N or K are not aligned.") */
  LLMMM_ERR_UNSUPPORTED = 2, /* dtype or device not supported ("T is not supported.") */
  LLMMM_ERR_CUDA        = 3, /* a CUDA runtime / driver call failed; see llmmm_last_error() */
  LLMMM_ERR_DEVICE_WAIT = 4  /* a bounded device-side wait ran out (llmmm_check_status) */
};

/* Text of the last error raised on the calling thread ("" if none). */
const char* llmmm_last_error(void);

/* Library version string. */
const char* llmmm_version(void);

/* C[M,N] = A[M,K] * B[K,N]; A, B, C row-major half; fp32 accumulation, one
 * round-to-nearest conversion of the result.
 * Replaces LLMMM::fp16_mm<half> (src/mm/fp16/mm.h:9-10, launcher
 * src/mm/fp16/mm.cu:7-42).  The reference accepts only M%256 == N%256 == 0,
 * K%16 == 0; this library accepts any M >= 1 with N%8 == 0 and K%8 == 0
 * (16-byte row pitch) and 16-byte aligned base pointers. */
int llmmm_fp16_mm_f16(const void* A, const void* B, void* C, int M, int N, int K, llmmm_stream_t stream);

/* Same for __nv_bfloat16: LLMMM::fp16_mm<__nv_bfloat16> (src/mm/fp16/mm.cu:45-46). */
int llmmm_fp16_mm_bf16(const void* A, const void* B, void* C, int M, int N, int K, llmmm_stream_t stream);

/* FP8 e4m3 blockwise GEMM with fused 1x128 output quantisation.
 *   A            [M,K]          e4m3, row-major (K contiguous)
 *   A_scale_t    [(K/128), M]   fp32, one scale per row per 128-wide K group
 *   B_t          [N,K]          e4m3, row-major (K contiguous) = B transposed
 *   B_scale_t    [(N/128),(K/128)] fp32, one scale per 128x128 block
 *   C            [M,N]          e4m3 out
 *   C_scale_t    [(N/128), M]   fp32 out, one scale per row per 128-wide N group
 * acc[m,n] = sum_kb ( sum_{k in kb} A*B ) * (A_scale_t[kb,m] * B_scale_t[n/128,kb]),
 * amax over each 1x128 group of acc, C_scale = amax/448, C = e4m3(acc * (448/amax)).
 * An all-zero group yields scale 0 and zeros (the reference yields NaN there).
 * Replaces the launchers generated at examples/005.fp8.mm.cu:2466-2577, e.g.
 * fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8__opt_reg
 * (same argument order).  Requires N%128 == 0, K%128 == 0; any M >= 1
 * (the reference requires M%128 == 0).  M <= 64 takes a split-K path; some
 * shapes need a caller-owned workspace for it (see llmmm_set_workspace), without
 * one those shapes run on the general kernel. */
int llmmm_fp8_blockwise_mm_e4m3out(const void*    A,
                                   const float*   A_scale_t,
                                   const void*    B_t,
                                   const float*   B_scale_t,
                                   void*          C,
                                   float*         C_scale_t,
                                   int            M,
                                   int            N,
                                   int            K,
                                   llmmm_stream_t stream);

/* N-split across GPUs with the all-gather of the outputs fused into the GEMM: this call computes the column
 * shard [col_offset, col_offset + N) of a product that is N_total columns wide (B_t / B_scale_t are this
 * rank's slabs: [N, K] and [(N/128), (K/128)]) and stores the shard into the FULL outputs
 * C [M, N_total] e4m3 and C_scale_t [(N_total/128), M] of n_dsts (1..8) destinations: this GPU's own buffers
 * and the other GPUs' buffers mapped into this GPU's address space (virtual-memory API or peer access).  The peer stores are plain
 * stores issued by the epilogue while other tiles are still being computed; when the kernel has completed on
 * every rank (stream order + a barrier between the ranks) every destination holds the whole C.  The reference
 * has no multi-GPU code.  Shapes as for llmmm_fp8_blockwise_mm_e4m3out; N_total, col_offset multiples of 128. */
int llmmm_fp8_blockwise_mm_e4m3out_gather(const void*    A,
                                          const float*   A_scale_t,
                                          const void*    B_t,
                                          const float*   B_scale_t,
                                          void* const*   C_dsts,
                                          float* const*  C_scale_dsts,
                                          int            n_dsts,
                                          int            N_total,
                                          int            col_offset,
                                          int            M,
                                          int            N,
                                          int            K,
                                          llmmm_stream_t stream);

/* gate_up projection with the SwiGLU epilogue fused (the reference's README.md:16 plans this fusion; it has
 * no implementation of it):
 *   B_gate_up_t  [2I, K]  e4m3: rows 0..I-1 the gate projection, rows I..2I-1 the up projection
 *   B_scale_t    [(2I/128), (K/128)] fp32
 *   acc = the blockwise product of llmmm_fp8_blockwise_mm_e4m3out, [M, 2I], kept on chip
 *   h[m, i] = silu(acc[m, i]) * acc[m, I + i],  silu(x) = x / (1 + exp(-x))   (fp32)
 *   H [M, I] e4m3 and H_scale_t [(I/128), M]: h quantised in 1x128 groups along I by the same rule as C above,
 *   which is the A / A_scale_t format of the down projection that consumes it.
 * Requires I%128 == 0, K%128 == 0, any M >= 1.  M > 64 runs one fused kernel (256-row tiles).  M <= 64 runs the
 * weight-streaming decode kernel into scratch followed by a small SwiGLU + quantisation kernel, provided the
 * registered scratch (llmmm_set_workspace) has llmmm_fp8_swiglu_workspace_bytes(M, I, K) bytes; otherwise the
 * 256-row kernel runs for small M too (same results up to the order of fp32 sums, several times slower). */
int llmmm_fp8_blockwise_mm_swiglu_e4m3out(const void*    A,
                                          const float*   A_scale_t,
                                          const void*    B_gate_up_t,
                                          const float*   B_scale_t,
                                          void*          H,
                                          float*         H_scale_t,
                                          int            M,
                                          int            I,
                                          int            K,
                                          llmmm_stream_t stream);

size_t llmmm_fp8_swiglu_workspace_bytes(int M, int I, int K);

/* qkv projection with the per-head q/k RMSNorm and the rotary position embedding fused in front of the output
 * quantisation (the reference's README.md:16 plans "norm/rope fusion"; it has no implementation of it).  Heads
 * are 128 columns wide, which is exactly one 1x128 quantisation group:
 *   B_t [N, K] e4m3 with N = (n_q_heads + 2 n_kv_heads) * 128: query heads first, then key heads, then value heads
 *   acc = the blockwise product of llmmm_fp8_blockwise_mm_e4m3out, [M, N], kept on chip
 *   query / key head x (128 values of row m):
 *     if the weight pointer of its kind is not NULL:  x[i] = x[i] * (1 / sqrt(mean(x^2) + eps)) * weight[i]
 *     p = positions[m];  for i < 64:  y[i]      = x[i]      * cos_table[p, i] - x[i + 64] * sin_table[p, i]
 *                                     y[i + 64] = x[i + 64] * cos_table[p, i] + x[i]      * sin_table[p, i]
 *   value heads pass unchanged; every head is then quantised as one 1x128 group into C [M, N] e4m3 and
 *   C_scale_t [(N/128), M] by the same rule as C above.
 *   positions [M] int32 (rows of the angle tables), cos_table / sin_table [table_rows, 64] fp32, weights [128] fp32.
 *   A position outside [0, table_rows) is clamped to the nearest row (no access outside the tables is made) and
 *   recorded: llmmm_check_status then returns LLMMM_ERR_DEVICE_WAIT with code 0x201.
 * Requires K%128 == 0, any M >= 1; tables, weights, A, B_t and C 16-byte aligned.  M > 64 runs one fused kernel
 * (256-row tiles, always whole: registered scratch is not used).  M <= 64 runs the
 * weight-streaming decode kernel into scratch followed by a small kernel, provided the registered scratch has
 * llmmm_fp8_qk_norm_rope_workspace_bytes(M, N, K) bytes; otherwise the 256-row kernel runs for small M too. */
int llmmm_fp8_blockwise_mm_qk_norm_rope_e4m3out(const void*    A,
                                                const float*   A_scale_t,
                                                const void*    B_t,
                                                const float*   B_scale_t,
                                                void*          C,
                                                float*         C_scale_t,
                                                const int*     positions,
                                                const float*   cos_table,
                                                const float*   sin_table,
                                                int            table_rows,
                                                const float*   q_norm_weight,
                                                const float*   k_norm_weight,
                                                float          eps,
                                                int            n_q_heads,
                                                int            n_kv_heads,
                                                int            M,
                                                int            N,
                                                int            K,
                                                llmmm_stream_t stream);

size_t llmmm_fp8_qk_norm_rope_workspace_bytes(int M, int N, int K);

/* Same product with the fp32 accumulator written out unquantised, C [M,N] fp32.
 * Replaces fp8_gemm_blockwise_quant_A_1x128__B_128x128__output_fp32
 * (examples/005.fp8.mm.cu:217-246). */
int llmmm_fp8_blockwise_mm_f32out(const void*    A,
                                  const float*   A_scale_t,
                                  const void*    B_t,
                                  const float*   B_scale_t,
                                  float*         C,
                                  int            M,
                                  int            N,
                                  int            K,
                                  llmmm_stream_t stream);

/* Activation quantiser: x [M,K] fp32 -> q [M,K] e4m3, scale [(K/128), M] fp32.
 * Per row and 128-wide K group: s = amax/448, q = e4m3(s ? x/s : 0).
 * Replaces fp8_blockwise_symmetric_quantization<1,128,true>
 * (examples/005.fp8.mm.cu:439-500, launcher :547-563).  Requires K%128 == 0. */
int llmmm_fp8_quant_1x128(const float* x, void* q, float* scale, int M, int K, llmmm_stream_t stream);

/* RMSNorm fused in front of the activation quantiser (the reference's README.md:16 plans RMSNorm hooks; it
 * has no implementation): y[m,k] = x[m,k] * rsqrt(mean_k(x[m,:]^2) + eps) * weight[k] in fp32, then y is
 * quantised exactly as llmmm_fp8_quant_1x128 quantises x: q [M,K] e4m3, scale [(K/128), M].  One pass over x
 * from HBM instead of three (normalise, write, re-read to quantise).  Requires K%128 == 0, eps >= 0. */
int llmmm_fp8_rmsnorm_quant_1x128(const float* x, const float* weight, float eps, void* q, float* scale, int M, int K,
                                  llmmm_stream_t stream);

/* Weight quantiser: x [rows,cols] fp32 -> q [rows,cols] e4m3,
 * scale [(rows/128),(cols/128)] fp32, one scale per 128x128 block.
 * Replaces fp8_blockwise_symmetric_quantization<128,128,false>
 * (examples/005.fp8.mm.cu:503-544).  Requires rows%128 == 0, cols%128 == 0. */
int llmmm_fp8_quant_128x128(const float* x, void* q, float* scale, int rows, int cols, llmmm_stream_t stream);

/* dst[N,M] = src[M,N] transposed, elements of 1 byte (e4m3) or 4 bytes (float).
 * Replaces LLMMM::transpose_matrix__aligned_128<T> (src/base/base.h:8-9, src/base/base.cu:125-155), used
 * to build B_transposed[N,K] from B[K,N] (examples/005.fp8.mm.cu:2657-2660).  Requires M%128 == 0 and
 * N%128 == 0 ("M or N can't be divided 128." otherwise), elem_bytes 1 or 4. */
int llmmm_transpose_aligned_128(void* dst, const void* src, int M, int N, int elem_bytes, llmmm_stream_t stream);

/* Split-K scratch.  The reference has no split-K (README.md:22 lists it as to
 * do) and its launchers allocate nothing, so the scratch is caller-owned: bytes
 * needed for a given problem, and registration of a device buffer for the
 * current device.  Two paths use it: the decode-sized (M <= 64) FP8 kernel, and,
 * for M > 128, the FP8 and FP16/BF16 kernels when their last wave of 256x256
 * tiles would leave most of the GPU idle: those tiles are then cut along K, the
 * fp32 partial tiles go through the scratch and are added in a fixed order
 * (results are bitwise stable from call to call, and differ from the unsplit
 * ones only by the association of fp32 sums).  llmmm_fp8_workspace_bytes gives
 * the size for an FP8 problem; for FP16/BF16 pass the same M (any N, K >= 128).
 * Without registered scratch every shape still runs, unsplit.  llmmm_set_workspace
 * clears the parts of the buffer that must be zero between launches (it
 * synchronises; register once, outside the token loop); every launch leaves them
 * zero again.  One buffer per device serves all later calls on that device, so
 * calls that use the registered scratch must be serialised per device (one
 * stream, or events between streams). */
size_t llmmm_fp8_workspace_bytes(int M, int N, int K);
int    llmmm_set_workspace(void* device_ptr, size_t bytes);

/* The same scratch as an explicit argument, for hosts with several streams or threads: the call uses `workspace`
 * (llmmm_fp8_workspace_bytes bytes, 256-byte aligned; NULL with 0 bytes = this call runs without scratch) and never
 * looks at the buffer registered for the device, so which kernel runs depends on the arguments alone, and two
 * streams with two buffers may overlap freely.  A buffer must be prepared once before its first use, and again
 * after llmmm_check_status reported an expired wait: llmmm_prepare_workspace clears, asynchronously on `stream`,
 * the parts that have to be zero between launches (every launch leaves them zero again).  No counterpart in
 * the reference (it has no split-K, README.md:22). */
int llmmm_prepare_workspace(void* workspace, size_t workspace_bytes, llmmm_stream_t stream);
int llmmm_fp8_blockwise_mm_e4m3out_ws(const void*    A,
                                      const float*   A_scale_t,
                                      const void*    B_t,
                                      const float*   B_scale_t,
                                      void*          C,
                                      float*         C_scale_t,
                                      int            M,
                                      int            N,
                                      int            K,
                                      void*          workspace,
                                      size_t         workspace_bytes,
                                      llmmm_stream_t stream);
int llmmm_fp8_blockwise_mm_f32out_ws(const void*    A,
                                     const float*   A_scale_t,
                                     const void*    B_t,
                                     const float*   B_scale_t,
                                     float*         C,
                                     int            M,
                                     int            N,
                                     int            K,
                                     void*          workspace,
                                     size_t         workspace_bytes,
                                     llmmm_stream_t stream);
int llmmm_fp16_mm_f16_ws(const void* A, const void* B, void* C, int M, int N, int K, void* workspace, size_t workspace_bytes,
                         llmmm_stream_t stream);
int llmmm_fp16_mm_bf16_ws(const void* A, const void* B, void* C, int M, int N, int K, void* workspace, size_t workspace_bytes,
                          llmmm_stream_t stream);
/* For every other entry point (the fused hooks, llmmm_describe_plan, llmmm_tune): binds `workspace` to the CALLING
 * THREAD; until it is unbound (NULL, 0) every call this thread makes uses it instead of the registered buffer.
 * One host thread per stream, each with its own bound buffer, is race-free. */
int llmmm_bind_workspace(void* workspace, size_t workspace_bytes);

/* A promise about the B_t / B_scale_t operands of later FP8 GEMM calls from this process: they are model
 * weights, never written by the kernel that runs immediately before the GEMM on the same stream.  With it
 * (enabled != 0) a decode-sized call (M <= 64) requests its first weight tiles while the preceding kernel of
 * the stream is still finishing (programmatic dependent launch; activations, scales and outputs still wait
 * for that kernel).  Off by default: then nothing is read before the preceding kernel has completed.  No
 * counterpart in the reference. */
int llmmm_set_static_weights(int enabled);

/* Decode-sized FP8 blockwise GEMM for callers that cannot provide scratch memory.
 * This one has no counterpart in the reference (which has neither split-K nor
 * any scratch).  It exists for hosts where device allocation is off the table:
 * servers whose own pool already holds all of device memory, and token loops
 * that must never reach cudaMalloc/cudaFree because those calls synchronise the
 * device.  Same arguments and results as llmmm_fp8_blockwise_mm_e4m3out, but the
 * split-K scratch is a fixed 2,621,440-byte array inside the library image (held
 * by every GPU that loads the library until the process exits), so:
 *   - 1 <= M <= 16 and N <= 524288 only; anything larger returns
 *     LLMMM_ERR_SHAPE with a message naming the limit;
 *   - no call allocates or frees anything; the first call on a device looks up
 *     the array's device address (make that first call outside stream capture);
 *   - all calls on a device share the one array, which every completed call
 *     leaves all zero again: two calls whose kernels can overlap on the GPU
 *     (different streams) race; serialise them. */
int llmmm_fp8_blockwise_mm_e4m3out_noalloc(const void*    A,
                                           const float*   A_scale_t,
                                           const void*    B_t,
                                           const float*   B_scale_t,
                                           void*          C,
                                           float*         C_scale_t,
                                           int            M,
                                           int            N,
                                           int            K,
                                           llmmm_stream_t stream);

/* Reads the device status word of the current device after synchronising
 * `stream`.  Returns LLMMM_OK, or LLMMM_ERR_DEVICE_WAIT with the code of the
 * wait that ran out in llmmm_last_error(); the word is cleared. */
int llmmm_check_status(llmmm_stream_t stream);

/* Failure-detection self-test: runs a one-CTA kernel whose only wait is on a barrier that nothing signals,
 * with a limit of `limit_us` microseconds, and synchronises.  Returns LLMMM_OK when the kernel gave up the
 * wait and ran to its normal end; the expiry is then visible through llmmm_check_status(), which returns
 * LLMMM_ERR_DEVICE_WAIT (code 0x1ff) once and clears the word.  Nothing faults or hangs.  The reference has
 * no counterpart (its kernels contain no waits on other agents). */
int llmmm_selftest_wait_expiry(unsigned int limit_us, llmmm_stream_t stream);

/* Problem kinds for the two calls below. */
#define LLMMM_KIND_FP16 0
#define LLMMM_KIND_BF16 1
#define LLMMM_KIND_FP8_E4M3OUT 2
#define LLMMM_KIND_FP8_F32OUT 3

/* Which kernel, tiling, wave count, split-K or cluster choice a call with these sizes would get on the current
 * device with the scratch registered right now, as one line of text (NUL-terminated, truncated to len).
 * Nothing is launched.  The reference has no heuristics (one fixed tile, src/mm/fp16/mm.cu:9-14; README.md:22
 * lists auto-tuning as to do). */
int llmmm_describe_plan(int kind, int M, int N, int K, char* buf, size_t len);

/* The tune(N, K) member of the reference's planned functor (MM_IMPL<T>::tune, src/mm/fp32/impl.h:20, a stub
 * there).  Here the per-shape choices are closed-form, so tuning is the one-time per-device set-up: function
 * attributes of every kernel of the family and the cluster occupancy queries, so that the first real call
 * (possibly inside a latency-critical loop or a stream capture) pays none of it.
 * For the two FP8 kinds it also SEARCHES: the plans of the decode-sized kernel that fit an [N, K] weight (stream-K
 * through the scratch registered or bound at the time, clusters of 2..7 CTAs per output group) are timed with
 * CUDA events at M = 16, 32 and 64 over weight copies that exceed the L2 cache, and the winner is recorded per
 * (device, M bucket, N, K); later calls with that weight shape use it and llmmm_describe_plan says "measured by
 * llmmm_tune".  With the scratch registered it also times, at M = 128, the single-CTA kernel against the pair
 * kernel and records which of the two calls of 65..128 rows with this weight shape get.  The search allocates and frees temporary operands (about 256 MB) and synchronises: call it at
 * set-up, once per weight shape, after registering the scratch.  It also touches the decode kernels' module and
 * looks up the built-in scratch of llmmm_fp8_blockwise_mm_e4m3out_noalloc, so a host that later hands all device
 * memory to its own pool should call it (or one no-alloc call) before doing so. */
int llmmm_tune(int kind, int N, int K);

/* Number of kernels launched by this library in the calling process. */
uint64_t llmmm_launch_count(void);

/* How many of those launches cut the tiles of their last wave along K (possible for M > 128 once scratch
 * is registered with llmmm_set_workspace; see there).  A diagnostic: lets a caller see that its scratch
 * registration took effect.  No counterpart in the reference. */
uint64_t llmmm_split_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* LLMMM_C_H */
