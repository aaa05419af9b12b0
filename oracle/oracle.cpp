// CPU oracle for the LLMMM GEMM hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the host, the arithmetic of the reference's GPU
// reference GEMMs and of its FP8 blockwise quantisation rules.  It is the
// checker used by the test-suite, by the smoke check and by the CPU-baseline
// leg of the benchmark; the product library never links or calls it.
//
// Parity status: the reference ships no golden vectors for this path.  The
// restatement is pinned against the reference's own kernels executed on a
// B200 (see oracle/pin_against_ref.py and tests/golden/ref_pins.json).
//
// Every function cites the reference file:line it follows (paths relative to
// the reference project root).  Build: see oracle/Makefile
// (-ffp-contract=off, no fast-math; FMAs are written explicitly where the
// reference's nvcc build contracts them).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <omp.h>
#include <vector>

namespace {

float g_e4m3_lut[256];
bool  g_lut_ready = false;

// e4m3 byte -> float, exact (every e4m3 value is representable in fp16).
void build_lut()
{
  if (g_lut_ready) {
    return;
  }
  for (int i = 0; i < 256; ++i) {
    __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)i, __NV_E4M3);
    __half     h(hr);
    g_e4m3_lut[i] = __half2float(h);
  }
  g_lut_ready = true;
}

// float -> e4m3 byte with the semantics of the `__nv_fp8_e4m3(float)`
// constructor the reference uses everywhere (examples/005.fp8.mm.cu:481,
// 1125): round-to-nearest-even, saturate to +-448, NaN -> 0x7f.
inline uint8_t enc_e4m3(float x)
{
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

}  // namespace

extern "C" {

int oracle_num_threads()
{
  return omp_get_max_threads();
}

void oracle_set_num_threads(int n)
{
  if (n > 0) {
    omp_set_num_threads(n);
  }
}

// ---------------------------------------------------------------- codecs --

void oracle_e4m3_decode(const uint8_t* q, float* out, int64_t n)
{
  build_lut();
  for (int64_t i = 0; i < n; ++i) {
    out[i] = g_e4m3_lut[q[i]];
  }
}

void oracle_e4m3_encode(const float* x, uint8_t* out, int64_t n)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    out[i] = enc_e4m3(x[i]);
  }
}

// fp32 -> fp16 / bf16 bits, round-to-nearest-even: the `T(float)` constructor
// used by test/fp16_mm_test.cc:40-45 to prepare inputs and by
// src/mm/fp16/mm.cuh:427 for the single output rounding.
void oracle_f32_to_f16(const float* x, uint16_t* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) {
    __half h = __float2half_rn(x[i]);
    std::memcpy(&out[i], &h, 2);
  }
}

void oracle_f16_to_f32(const uint16_t* x, float* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) {
    __half h;
    std::memcpy(&h, &x[i], 2);
    out[i] = __half2float(h);
  }
}

void oracle_f32_to_bf16(const float* x, uint16_t* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) {
    __nv_bfloat16 h = __float2bfloat16_rn(x[i]);
    std::memcpy(&out[i], &h, 2);
  }
}

void oracle_bf16_to_f32(const uint16_t* x, float* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) {
    uint32_t u = (uint32_t)x[i] << 16;
    std::memcpy(&out[i], &u, 4);
  }
}

// ------------------------------------------------------- reference GEMMs --

// test/kahan.cu:7-27.  A[M,K], B[K,N], C[M,N] row-major fp32.  The reference
// is compiled by nvcc with its default -fmad=true, so `A[k]*B[k*N] - diff`
// is one fused multiply-add; it is written as fmaf here.  `row0/rows` select
// a slab of C rows so that large shapes can be sampled.
void oracle_kahan_gemm(const float* A, const float* B, float* C, int M, int N, int K, int row0, int rows)
{
  (void)M;
#pragma omp parallel for schedule(dynamic, 1)
  for (int mi = 0; mi < rows; ++mi) {
    const int          m = row0 + mi;
    std::vector<float> sum(N, 0.0f), diff(N, 0.0f);
    const float*       a = A + (int64_t)m * K;
    for (int k = 0; k < K; ++k) {
      const float  av = a[k];
      const float* b  = B + (int64_t)k * N;
      for (int n = 0; n < N; ++n) {
        float y = fmaf(av, b[n], -diff[n]);
        float t = sum[n] + y;
        diff[n] = (t - sum[n]) - y;
        sum[n]  = t;
      }
    }
    std::memcpy(C + (int64_t)mi * N, sum.data(), sizeof(float) * N);
  }
}

// test/kahan.cu:39-56.  `sum += A[k] * B[k*N]` with `double sum`: the product
// is an fp32 multiply (one rounding) that is then widened and added in fp64.
void oracle_double_gemm(const float* A, const float* B, float* C, int M, int N, int K, int row0, int rows)
{
  (void)M;
#pragma omp parallel for schedule(dynamic, 1)
  for (int mi = 0; mi < rows; ++mi) {
    const int           m = row0 + mi;
    std::vector<double> sum(N, 0.0);
    const float*        a = A + (int64_t)m * K;
    for (int k = 0; k < K; ++k) {
      const float  av = a[k];
      const float* b  = B + (int64_t)k * N;
      for (int n = 0; n < N; ++n) {
        float p = av * b[n];
        sum[n] += (double)p;
      }
    }
    float* c = C + (int64_t)mi * N;
    for (int n = 0; n < N; ++n) {
      c[n] = (float)sum[n];
    }
  }
}

// Ground truth for the FP16/BF16 GEMM (src/mm/fp16/mm.cuh:85,267-274,427
// computes sum_k float(A)*float(B) in fp32 and rounds once): exact fp64
// accumulation of exact products of the already-rounded inputs (given here
// as fp32 values that are exactly representable in the 16-bit type).
void oracle_exact_gemm_f64(const float* A, const float* B, double* C, int M, int N, int K, int row0, int rows)
{
  (void)M;
#pragma omp parallel for schedule(dynamic, 1)
  for (int mi = 0; mi < rows; ++mi) {
    const int           m = row0 + mi;
    std::vector<double> sum(N, 0.0);
    const float*        a = A + (int64_t)m * K;
    for (int k = 0; k < K; ++k) {
      const double av = a[k];
      const float* b  = B + (int64_t)k * N;
      for (int n = 0; n < N; ++n) {
        sum[n] += av * (double)b[n];
      }
    }
    std::memcpy(C + (int64_t)mi * N, sum.data(), sizeof(double) * N);
  }
}

// ------------------------------------------------------------ quantisers --

// Activation quantiser, examples/005.fp8.mm.cu:439-500 instantiated as
// <1,128,SCALE_TRANSPOSE=true> (call site :2686).  x[M,K] fp32 ->
// q[M,K] e4m3, scale[(K/128), M] fp32.  Per row and per group of 128
// consecutive k: amax = max|x| (:472-478), s = amax/448 (:479),
// q = e4m3(s ? x/s : 0) (:481-486), scale[g*M+m] = s (:493-494).
// K must be a multiple of 128 (the reference reads whole 128-wide rows).
void oracle_quant_1x128(const float* x, uint8_t* q, float* scale, int M, int K)
{
  const int G = K / 128;
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    for (int g = 0; g < G; ++g) {
      const float* xp   = x + (int64_t)m * K + g * 128;
      float        amax = 0.0f;
      for (int i = 0; i < 128; ++i) {
        float a = std::fabs(xp[i]);
        amax    = (amax < a) ? a : amax;
      }
      const float s  = amax / 448.0f;
      uint8_t*    qp = q + (int64_t)m * K + g * 128;
      for (int i = 0; i < 128; ++i) {
        qp[i] = enc_e4m3(s ? xp[i] / s : 0.0f);
      }
      scale[(int64_t)g * M + m] = s;
    }
  }
}

// Weight quantiser, examples/005.fp8.mm.cu:503-544 instantiated as
// <128,128,false> on B_transposed[N,K] (call site :2739).  Per 128x128 block:
// amax over the block (:504-515), s = amax/448 (:516), q = e4m3(s ? x/s : 0)
// (:523-528), scale[(r/128)*(cols/128) + c/128] = s (:538-540).
// rows, cols multiples of 128.
void oracle_quant_128x128(const float* x, uint8_t* q, float* scale, int rows, int cols)
{
  const int RB = rows / 128, CB = cols / 128;
#pragma omp parallel for schedule(static) collapse(2)
  for (int rb = 0; rb < RB; ++rb) {
    for (int cb = 0; cb < CB; ++cb) {
      float amax = 0.0f;
      for (int r = 0; r < 128; ++r) {
        const float* xp = x + (int64_t)(rb * 128 + r) * cols + cb * 128;
        for (int c = 0; c < 128; ++c) {
          float a = std::fabs(xp[c]);
          amax    = (amax < a) ? a : amax;
        }
      }
      const float s = amax / 448.0f;
      for (int r = 0; r < 128; ++r) {
        const float* xp = x + (int64_t)(rb * 128 + r) * cols + cb * 128;
        uint8_t*     qp = q + (int64_t)(rb * 128 + r) * cols + cb * 128;
        for (int c = 0; c < 128; ++c) {
          qp[c] = enc_e4m3(s ? xp[c] / s : 0.0f);
        }
      }
      scale[(int64_t)rb * CB + cb] = s;
    }
  }
}

// ------------------------------------------------- FP8 blockwise GEMM -----

// fp32 accumulator of the blockwise GEMM, before C is re-quantised.
//   A_q[M,K], B_q[N,K] e4m3 bytes (both K-contiguous),
//   A_s[(K/128), M], B_s[(N/128), (K/128)] fp32, acc[rows, N] fp32.
// examples/005.fp8.mm.cu:1057-1068: per 128-K block the scale is
// sc = A_s[kb*M+m] * B_s[nb*(K/128)+kb], rounded once to fp32;
// :890-901 (CAL_ON_LAST): acc += p * sc, one FMA under nvcc's default
// contraction, where p is the fp32 tensor-core sum of the block's 128 exact
// products.  mode 0 ("T1"): p accumulated in fp32, ascending k.
// mode 1 ("T0"): p accumulated exactly in fp64 and the promotion done in
// fp64 as well (ground truth for the quantised operands).
void oracle_fp8_blockwise_acc(const uint8_t* A_q,
                              const float*   A_s,
                              const uint8_t* B_q,
                              const float*   B_s,
                              float*         acc_f32,
                              double*        acc_f64,
                              int            M,
                              int            N,
                              int            K,
                              int            row0,
                              int            rows,
                              int            mode)
{
  build_lut();
  const int          KB = K / 128;
  std::vector<float> Bf((int64_t)N * K);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)N * K; ++i) {
    Bf[i] = g_e4m3_lut[B_q[i]];
  }
#pragma omp parallel for schedule(dynamic, 1)
  for (int mi = 0; mi < rows; ++mi) {
    const int          m = row0 + mi;
    std::vector<float> a(K);
    for (int k = 0; k < K; ++k) {
      a[k] = g_e4m3_lut[A_q[(int64_t)m * K + k]];
    }
    for (int n = 0; n < N; ++n) {
      const int    nb = n / 128;
      const float* b  = Bf.data() + (int64_t)n * K;
      if (mode == 0) {
        float acc = 0.0f;
        for (int kb = 0; kb < KB; ++kb) {
          float p = 0.0f;
          for (int k = kb * 128; k < kb * 128 + 128; ++k) {
            p += a[k] * b[k];  // exact product, fp32 running sum
          }
          const float sc = A_s[(int64_t)kb * M + m] * B_s[(int64_t)nb * KB + kb];
          acc            = fmaf(p, sc, acc);
        }
        acc_f32[(int64_t)mi * N + n] = acc;
      }
      else {
        double acc = 0.0;
        for (int kb = 0; kb < KB; ++kb) {
          double p = 0.0;
          for (int k = kb * 128; k < kb * 128 + 128; ++k) {
            p += (double)a[k] * (double)b[k];
          }
          const double sc = (double)A_s[(int64_t)kb * M + m] * (double)B_s[(int64_t)nb * KB + kb];
          acc += p * sc;
        }
        acc_f64[(int64_t)mi * N + n] = acc;
      }
    }
  }
}

// Fused C re-quantisation, examples/005.fp8.mm.cu:1107-1138 (the rule of all
// kernels after the first): per row m and 128-wide column block nb,
// amax = max|acc|, scale = amax/448, scale_inv = 448/amax,
// C_q = e4m3(acc*scale_inv), C_s[nb*ldcs + m] = scale.
// The reference has no guard for an all-zero group (0*inf = NaN there);
// this library defines that case as scale = 0, q = 0, and so does the oracle.
// acc is [rows, N]; C_s is written at column row0+mi of a [(N/128), ldcs] array.
void oracle_c_quant_1x128(const float* acc, uint8_t* C_q, float* C_s, int rows, int N, int ldcs, int row0)
{
  const int NB = N / 128;
#pragma omp parallel for schedule(static)
  for (int mi = 0; mi < rows; ++mi) {
    for (int nb = 0; nb < NB; ++nb) {
      const float* ap   = acc + (int64_t)mi * N + nb * 128;
      float        amax = 0.0f;
      for (int i = 0; i < 128; ++i) {
        amax = std::fmax(amax, std::fabs(ap[i]));
      }
      const float scale     = amax / 448.0f;
      const float scale_inv = (amax > 0.0f) ? 448.0f / amax : 0.0f;
      uint8_t*    qp        = C_q + (int64_t)mi * N + nb * 128;
      for (int i = 0; i < 128; ++i) {
        qp[i] = enc_e4m3(ap[i] * scale_inv);
      }
      C_s[(int64_t)nb * ldcs + row0 + mi] = scale;
    }
  }
}

// De-quantisation used by the reference's checks (examples/005.fp8.mm.cu:
// 2865-2869): float(C_q[m*N+n]) * C_s[(n/128)*M + m].
void oracle_dequant_1x128(const uint8_t* q, const float* s, float* out, int M, int N)
{
  build_lut();
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      out[(int64_t)m * N + n] = g_e4m3_lut[q[(int64_t)m * N + n]] * s[(int64_t)(n / 128) * M + m];
    }
  }
}

// src/base/base.cu:125-152 (`transpose_matrix__aligned_128`): out[N,M] = in[M,N]^T
// for 1-byte or 4-byte elements.
void oracle_transpose(const void* in, void* out, int M, int N, int elem_size)
{
  const uint8_t* src = (const uint8_t*)in;
  uint8_t*       dst = (uint8_t*)out;
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      std::memcpy(dst + ((int64_t)n * M + m) * elem_size, src + ((int64_t)m * N + n) * elem_size, elem_size);
    }
  }
}

}  // extern "C"
