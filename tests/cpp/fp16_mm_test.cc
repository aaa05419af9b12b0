// Harness driver in the shape of the reference's test/fp16_mm_test.cc:8-105:
// generate A[M,K], B[K,N], run LLMMM::fp16_mm<half> several times through the
// drop-in header, compare with a reference GEMM, print the error.  Differences
// from the reference driver: inputs are seeded, the comparison is against the
// oracle's Kahan GEMM of the rounded inputs (test/kahan.cu:7-27 restated on the
// host) on sampled rows, there is a pass/fail exit code, and the launches are
// timed with CUDA events.
//
// usage: fp16_mm_test [M N K]   (default 4096 4096 4096)
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "mm/fp16/mm.h"
#include "mm/mm_impl.h"
#include "../../oracle/oracle.h"

#define CHECK(call)                                                                                                    \
  do {                                                                                                                 \
    cudaError_t e = (call);                                                                                            \
    if (e != cudaSuccess) {                                                                                            \
      fprintf(stderr, "CUDA error: %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__);                         \
      return 2;                                                                                                        \
    }                                                                                                                  \
  } while (0)

int main(int argc, char** argv)
{
  int M = 4096, N = 4096, K = 4096;
  if (argc == 4) {
    M = atoi(argv[1]);
    N = atoi(argv[2]);
    K = atoi(argv[3]);
  }
  std::mt19937                          gen(0x4C4D4D4D);
  std::uniform_real_distribution<float> dis(-1.0f, 1.0f);
  std::vector<float>                    A((size_t)M * K), B((size_t)K * N);
  for (auto& v : A) v = dis(gen);
  for (auto& v : B) v = dis(gen);
  std::vector<uint16_t> Ah(A.size()), Bh(B.size()), Ch((size_t)M * N);
  oracle_f32_to_f16(A.data(), Ah.data(), (int64_t)A.size());
  oracle_f32_to_f16(B.data(), Bh.data(), (int64_t)B.size());
  oracle_f16_to_f32(Ah.data(), A.data(), (int64_t)A.size());  // the rounded inputs, as fp32
  oracle_f16_to_f32(Bh.data(), B.data(), (int64_t)B.size());

  half *dA, *dB, *dC;
  CHECK(cudaMalloc(&dA, Ah.size() * 2));
  CHECK(cudaMalloc(&dB, Bh.size() * 2));
  CHECK(cudaMalloc(&dC, Ch.size() * 2));
  CHECK(cudaMemcpy(dA, Ah.data(), Ah.size() * 2, cudaMemcpyDefault));
  CHECK(cudaMemcpy(dB, Bh.data(), Bh.size() * 2, cudaMemcpyDefault));
  CHECK(cudaMemset(dC, 0xff, Ch.size() * 2));

  // the reference launcher throws on misaligned shapes; so does the drop-in
  bool threw = false;
  try {
    LLMMM::fp16_mm(dA, dB, dC, M, N + 1, K, nullptr);
  }
  catch (const std::runtime_error& e) {
    threw = true;
  }
  if (!threw) {
    fprintf(stderr, "misaligned N was accepted\n");
    return 1;
  }

  cudaEvent_t e0, e1;
  CHECK(cudaEventCreate(&e0));
  CHECK(cudaEventCreate(&e1));
  for (int i = 0; i < 3; ++i) LLMMM::fp16_mm(dA, dB, dC, M, N, K, nullptr);
  CHECK(cudaEventRecord(e0));
  const int reps = 8;  // the reference driver launches 8 times (test/fp16_mm_test.cc:58-62)
  for (int i = 0; i < reps; ++i) LLMMM::fp16_mm(dA, dB, dC, M, N, K, nullptr);
  CHECK(cudaEventRecord(e1));
  CHECK(cudaDeviceSynchronize());
  float ms = 0;
  CHECK(cudaEventElapsedTime(&ms, e0, e1));
  CHECK(cudaMemcpy(Ch.data(), dC, Ch.size() * 2, cudaMemcpyDefault));

  std::vector<float> C(Ch.size());
  oracle_f16_to_f32(Ch.data(), C.data(), (int64_t)C.size());
  const int   rows_checked = M < 64 ? M : 64;
  const int   stride       = M / rows_checked;
  float       max_abs = 0, max_rel = 0;
  std::vector<float> ref(N);
  for (int r = 0; r < rows_checked; ++r) {
    const int m = r * stride;
    oracle_kahan_gemm(A.data(), B.data(), ref.data(), M, N, K, m, 1);
    for (int n = 0; n < N; ++n) {
      const float err = std::fabs(C[(size_t)m * N + n] - ref[n]);
      max_abs         = std::fmax(max_abs, err);
      if (std::fabs(ref[n]) > 0.05f * std::sqrt((float)K)) {
        max_rel = std::fmax(max_rel, err / std::fabs(ref[n]));
      }
    }
  }
  // the functor the reference plans (src/mm/fp32/impl.h): tune, run, verify against the result just checked
  LLMMM::MM_IMPL<half> impl;
  bool                 functor_ok = true;
  try {
    impl.tune(N, K);
    printf("plan: %s\n", impl.plan(M, N, K).c_str());
    impl.verify(dA, dB, dC, M, N, K);  // dC holds the product computed above
    std::vector<uint16_t> bad(Ch);
    bad[bad.size() / 2] ^= 0x4000;  // one corrupted element must be reported
    half* dBad;
    CHECK(cudaMalloc(&dBad, bad.size() * 2));
    CHECK(cudaMemcpy(dBad, bad.data(), bad.size() * 2, cudaMemcpyDefault));
    bool caught = false;
    try {
      impl.verify(dA, dB, dBad, M, N, K);
    }
    catch (const std::runtime_error&) {
      caught = true;
    }
    CHECK(cudaFree(dBad));
    functor_ok = caught;
  }
  catch (const std::runtime_error& e) {
    fprintf(stderr, "MM_IMPL: %s\n", e.what());
    functor_ok = false;
  }
  const double tflops = 2.0 * M * N * K / (ms / reps * 1e-3) / 1e12;
  printf("fp16_mm M=%d N=%d K=%d: %.1f us/launch, %.1f TFLOPS, max_abs_error = %.6f, max_relative_error = %.6f (%d rows vs Kahan)\n",
         M, N, K, ms / reps * 1e3, tflops, max_abs, max_rel, rows_checked);
  const bool ok = max_rel <= 1e-3f && functor_ok && llmmm_check_status(nullptr) == LLMMM_OK;
  printf("%s\n", ok ? "PASS" : "FAIL");
  return ok ? 0 : 1;
}
