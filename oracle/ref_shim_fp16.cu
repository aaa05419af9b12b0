// C entry points around the reference's own FP16 GEMM launcher, its two
// reference GEMM kernels and its transpose, so that the unmodified reference
// code (built for sm_100a by oracle/Makefile) can be called from the tests to
// pin the CPU oracle.  Test infrastructure only; not part of the product.
#include <stdexcept>

#include "base/base.h"   // reference: src/base/base.h
#include "kahan.h"       // reference: test/kahan.h
#include "mm/fp16/mm.h"  // reference: src/mm/fp16/mm.h

extern "C" {

int ref_kahan(const float* A, const float* B, float* C, int M, int N, int K)
{
  LLMMM::launch_kahan(A, B, C, M, N, K);
  return 0;
}

int ref_fp32_naive_mm(const float* A, const float* B, float* C, int M, int N, int K)
{
  LLMMM::launch_fp32_naive_mm(A, B, C, M, N, K);
  return 0;
}

int ref_fp16_mm_f16(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t s)
{
  try {
    LLMMM::fp16_mm<half>((const half*)A, (const half*)B, (half*)C, M, N, K, s);
  }
  catch (const std::runtime_error&) {
    return 1;
  }
  return 0;
}

int ref_fp16_mm_bf16(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t s)
{
  try {
    LLMMM::fp16_mm<__nv_bfloat16>((const __nv_bfloat16*)A, (const __nv_bfloat16*)B, (__nv_bfloat16*)C, M, N, K, s);
  }
  catch (const std::runtime_error&) {
    return 1;
  }
  return 0;
}

}  // extern "C"
