// Drop-in for the reference's src/mm/fp16/mm.h:9-10: same namespace, template
// and argument order.  The template forwards to the C ABI (include/llmmm_c.h)
// and turns a non-zero status into the std::runtime_error the reference
// launcher throws (src/mm/fp16/mm.cu:15-21).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "llmmm_c.h"

namespace LLMMM {

template<typename T>
void fp16_mm(const T* A, const T* B, T* C, int M, int N, int K, cudaStream_t stream)
{
  int rc;
  if (std::is_same<T, half>::value) {
    rc = llmmm_fp16_mm_f16(A, B, C, M, N, K, stream);
  }
  else if (std::is_same<T, __nv_bfloat16>::value) {
    rc = llmmm_fp16_mm_bf16(A, B, C, M, N, K, stream);
  }
  else {
    throw std::runtime_error("T is not supported.");
  }
  if (rc != LLMMM_OK) {
    throw std::runtime_error(std::string(llmmm_last_error()));
  }
}

}  // namespace LLMMM
