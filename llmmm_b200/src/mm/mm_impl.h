// The functor the reference plans for its GEMMs (src/mm/fp32/impl.h:12-29 declares MM_IMPL<float> with
// operator(), tune(N, K) and verify(A, B, benchmark, M, N, K), every body a stub that throws).  Here it is
// implemented for the 16-bit types the library computes in, over the C ABI (include/llmmm_c.h):
//   operator()  LLMMM::fp16_mm<T>
//   tune        llmmm_tune: one-time per-device set-up of the kernel family (the per-shape choices are
//               closed-form, llmmm_describe_plan prints them)
//   verify      runs the GEMM into a scratch C and compares it with `benchmark` on the host: relative error
//               1e-3 (plus one output ulp) with an absolute floor of 1e-3 * sqrt(K) / 8 for cancelling sums,
//               the gate of the parity tests; throws std::runtime_error naming the worst element otherwise.
#pragma once

#include <cmath>
#include <cstdio>
#include <vector>

#include "fp16/mm.h"

namespace LLMMM {

template<typename T>
class MM_IMPL {
public:
  void operator()(const T* A, const T* B, T* C, int M, int N, int K, cudaStream_t stream)
  {
    fp16_mm<T>(A, B, C, M, N, K, stream);
  }

  void tune(int N, int K)
  {
    throw_if(llmmm_tune(kind(), N, K));
  }

  // what the heuristics choose for (M, N, K) on the current device
  std::string plan(int M, int N, int K)
  {
    char buf[512];
    throw_if(llmmm_describe_plan(kind(), M, N, K, buf, sizeof(buf)));
    return buf;
  }

  void verify(const T* A, const T* B, const T* benchmark, int M, int N, int K)
  {
    T* C = nullptr;
    if (cudaMalloc(&C, sizeof(T) * (size_t)M * N) != cudaSuccess) {
      throw std::runtime_error("verify: cudaMalloc failed");
    }
    std::vector<T> got((size_t)M * N), want((size_t)M * N);
    try {
      (*this)(A, B, C, M, N, K, nullptr);
    }
    catch (...) {
      cudaFree(C);
      throw;
    }
    cudaError_t e = cudaMemcpy(got.data(), C, sizeof(T) * got.size(), cudaMemcpyDeviceToHost);
    cudaFree(C);
    if (e == cudaSuccess) {
      e = cudaMemcpy(want.data(), benchmark, sizeof(T) * want.size(), cudaMemcpyDefault);
    }
    if (e != cudaSuccess) {
      throw std::runtime_error(std::string("verify: ") + cudaGetErrorString(e));
    }
    const float out_ulp = std::is_same<T, half>::value ? 0x1p-11f : 0x1p-8f;
    const float floor_  = 1e-3f * std::sqrt((float)K) / 8.0f;
    for (size_t i = 0; i < got.size(); ++i) {
      const float g = to_float(got[i]), w = to_float(want[i]);
      if (!(std::fabs(g - w) <= (1e-3f + out_ulp) * std::fabs(w) + floor_)) {
        char msg[160];
        snprintf(msg, sizeof(msg), "verify: C[%zu,%zu] = %g, benchmark %g", i / N, i % N, g, w);
        throw std::runtime_error(msg);
      }
    }
  }

private:
  static int kind()
  {
    return std::is_same<T, half>::value ? LLMMM_KIND_FP16 : LLMMM_KIND_BF16;
  }

  static float to_float(half v)
  {
    return __half2float(v);
  }

  static float to_float(__nv_bfloat16 v)
  {
    return __bfloat162float(v);
  }

  static void throw_if(int rc)
  {
    if (rc != LLMMM_OK) {
      throw std::runtime_error(std::string(llmmm_last_error()));
    }
  }
};

}  // namespace LLMMM
