// C entry points around the reference's FP8 blockwise quantiser and GEMM
// launchers (examples/005.fp8.mm.cu, everything before its main()), built
// for sm_100a by oracle/Makefile.  Test infrastructure only.
#include REF_FP8_NOMAIN

#include <stdexcept>

#define REF_FP8_ENTRY(name, fn)                                                                                        \
  int name(const void*  A,                                                                                             \
           const float* A_s,                                                                                           \
           const void*  B,                                                                                             \
           const float* B_s,                                                                                           \
           void*        C,                                                                                             \
           float*       C_s,                                                                                           \
           int          M,                                                                                             \
           int          N,                                                                                             \
           int          K,                                                                                             \
           cudaStream_t s)                                                                                             \
  {                                                                                                                    \
    try {                                                                                                              \
      fn((const __nv_fp8_e4m3*)A, A_s, (const __nv_fp8_e4m3*)B, B_s, (__nv_fp8_e4m3*)C, C_s, M, N, K, s);              \
    }                                                                                                                  \
    catch (const std::runtime_error&) {                                                                                \
      return 1;                                                                                                        \
    }                                                                                                                  \
    return 0;                                                                                                          \
  }

extern "C" {

// activation quantiser <1,128,transposed scales> (examples/005.fp8.mm.cu:2686)
int ref_fp8_quant_1x128(const float* x, void* q, float* scale, int M, int K, cudaStream_t s)
{
  fp8_blockwise_symmetric_quantization<1, 128, true>(x, (__nv_fp8_e4m3*)q, scale, M, K, s);
  return 0;
}

REF_FP8_ENTRY(ref_fp8_mm_v1, fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8)
REF_FP8_ENTRY(ref_fp8_mm_opt_reg, fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8__opt_reg)
REF_FP8_ENTRY(ref_fp8_mm_inner_split,
              _fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8__opt_reg__quadra_buffer__inner_split)

int ref_fp8_mm_f32out(const void*  A,
                      const float* A_s,
                      const void*  B,
                      const float* B_s,
                      float*       C,
                      int          M,
                      int          N,
                      int          K,
                      cudaStream_t s)
{
  try {
    fp8_gemm_blockwise_quant_A_1x128__B_128x128__output_fp32(
      (const __nv_fp8_e4m3*)A, A_s, (const __nv_fp8_e4m3*)B, B_s, C, M, N, K, s);
  }
  catch (const std::runtime_error&) {
    return 1;
  }
  return 0;
}

}  // extern "C"
