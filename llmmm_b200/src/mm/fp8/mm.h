// FP8 blockwise GEMM and quantiser launchers under the names and signatures
// the reference generates in examples/005.fp8.mm.cu (launch macro :2466-2497,
// fp32-output launcher :217-225, quantiser :547-549).  All of the reference's
// fused-output variants compute the same function, so every name forwards to
// the one sm_100a implementation behind the C ABI (include/llmmm_c.h).  A
// non-zero status becomes the std::runtime_error the reference throws (:2490).
#pragma once

#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

#include "llmmm_c.h"

namespace LLMMM {

inline void throw_on_error(int rc)
{
  if (rc != LLMMM_OK) {
    throw std::runtime_error(std::string(llmmm_last_error()));
  }
}

}  // namespace LLMMM

#define LLMMM_FP8_LAUNCHER(name)                                                                                       \
  inline void name(const __nv_fp8_e4m3* A,                                                                             \
                   const float*         A_scale_transposed,                                                            \
                   const __nv_fp8_e4m3* B_transposed,                                                                  \
                   const float*         B_scale_transposed,                                                            \
                   __nv_fp8_e4m3*       C,                                                                             \
                   float*               C_scale_transposed,                                                            \
                   int                  M,                                                                             \
                   int                  N,                                                                             \
                   int                  K,                                                                             \
                   cudaStream_t         stream)                                                                        \
  {                                                                                                                    \
    LLMMM::throw_on_error(llmmm_fp8_blockwise_mm_e4m3out(                                                              \
      A, A_scale_transposed, B_transposed, B_scale_transposed, C, C_scale_transposed, M, N, K, stream));               \
  }

LLMMM_FP8_LAUNCHER(fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8)
LLMMM_FP8_LAUNCHER(fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8__opt_reg)
LLMMM_FP8_LAUNCHER(fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8__opt_reg__quadra_buffer__overlap_fma)
LLMMM_FP8_LAUNCHER(_fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8__opt_reg__quadra_buffer__inner_split)
#undef LLMMM_FP8_LAUNCHER

// The epilogue fusion the reference plans (README.md:16: SiLU * gate on the gate_up projection); named after
// the launchers above.  B_transposed is the gate_up weight [2I, K] with the gate rows first; C [M, I] and
// C_scale_transposed [(I/128), M] hold silu(gate) * up quantised 1x128 along I.
inline void fp8_gemm_blockwise_quant_A_1x128__B_128x128__swiglu__C_1x128__output_fp8(const __nv_fp8_e4m3* A,
                                                                                     const float*         A_scale_transposed,
                                                                                     const __nv_fp8_e4m3* B_transposed,
                                                                                     const float*         B_scale_transposed,
                                                                                     __nv_fp8_e4m3*       C,
                                                                                     float*               C_scale_transposed,
                                                                                     int                  M,
                                                                                     int                  I,
                                                                                     int                  K,
                                                                                     cudaStream_t         stream)
{
  LLMMM::throw_on_error(llmmm_fp8_blockwise_mm_swiglu_e4m3out(
    A, A_scale_transposed, B_transposed, B_scale_transposed, C, C_scale_transposed, M, I, K, stream));
}

// The other planned fusion (README.md:16: norm / rope): the qkv projection with heads of 128 columns (query heads,
// then key heads, then value heads); query and key heads are RMS-normalised per head (a null weight skips it) and
// rotated by the angle-table row positions[m] (pairs (i, i + 64)) before the 1x128 quantisation.
inline void fp8_gemm_blockwise_quant_A_1x128__B_128x128__qk_norm_rope__C_1x128__output_fp8(const __nv_fp8_e4m3* A,
                                                                                           const float*         A_scale_transposed,
                                                                                           const __nv_fp8_e4m3* B_transposed,
                                                                                           const float*         B_scale_transposed,
                                                                                           __nv_fp8_e4m3*       C,
                                                                                           float*               C_scale_transposed,
                                                                                           const int*           positions,
                                                                                           const float*         cos_table,
                                                                                           const float*         sin_table,
                                                                                           int                  table_rows,
                                                                                           const float*         q_norm_weight,
                                                                                           const float*         k_norm_weight,
                                                                                           float                eps,
                                                                                           int                  n_q_heads,
                                                                                           int                  n_kv_heads,
                                                                                           int                  M,
                                                                                           int                  N,
                                                                                           int                  K,
                                                                                           cudaStream_t         stream)
{
  LLMMM::throw_on_error(llmmm_fp8_blockwise_mm_qk_norm_rope_e4m3out(
    A, A_scale_transposed, B_transposed, B_scale_transposed, C, C_scale_transposed, positions, cos_table, sin_table,
    table_rows, q_norm_weight, k_norm_weight, eps, n_q_heads, n_kv_heads, M, N, K, stream));
}

inline void fp8_gemm_blockwise_quant_A_1x128__B_128x128__output_fp32(const __nv_fp8_e4m3* A,
                                                                     const float*         A_scale_transposed,
                                                                     const __nv_fp8_e4m3* B_transposed,
                                                                     const float*         B_scale_transposed,
                                                                     float*               C,
                                                                     int                  M,
                                                                     int                  N,
                                                                     int                  K,
                                                                     cudaStream_t         stream)
{
  LLMMM::throw_on_error(
    llmmm_fp8_blockwise_mm_f32out(A, A_scale_transposed, B_transposed, B_scale_transposed, C, M, N, K, stream));
}

// RMSNorm fused in front of the activation quantiser (README.md:16 plans the hook): q / scale as produced by
// fp8_blockwise_symmetric_quantization<1,128,true> for y = x * rsqrt(mean(x^2) + eps) * weight.
inline void fp8_rmsnorm_blockwise_symmetric_quantization_1x128(
  const float* x, const float* weight, float eps, __nv_fp8_e4m3* q, float* scale, int M, int K, cudaStream_t stream)
{
  LLMMM::throw_on_error(llmmm_fp8_rmsnorm_quant_1x128(x, weight, eps, q, scale, M, K, stream));
}

// Only the two instantiations the reference uses exist: <1,128,true>
// (activations, :2686) and <128,128,false> (weights, :2739).
template<int QUANT_M, int QUANT_N, bool SCALE_TRANPOSE>
void fp8_blockwise_symmetric_quantization(
  const float* x, __nv_fp8_e4m3* q, float* scale, int M, int N, cudaStream_t stream)
{
  static_assert(QUANT_N == 128 && ((QUANT_M == 1 && SCALE_TRANPOSE) || (QUANT_M == 128 && !SCALE_TRANPOSE)),
                "supported: <1,128,true> and <128,128,false>");
  if (QUANT_M == 1) {
    LLMMM::throw_on_error(llmmm_fp8_quant_1x128(x, q, scale, M, N, stream));
  }
  else {
    LLMMM::throw_on_error(llmmm_fp8_quant_128x128(x, q, scale, M, N, stream));
  }
}
