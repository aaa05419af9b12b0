// FP8 e4m3 blockwise symmetric quantisers for sm_100a (HBM-bound: 4 bytes read
// and 1 byte written per element).
//
// Replace the reference's fp8_blockwise_symmetric_quantization
// (examples/005.fp8.mm.cu:439-563): <1,128,true> for activations and
// <128,128,false> for weights.  The arithmetic is kept bit for bit:
// s = amax/448 (IEEE division), q = e4m3(s ? x/s : 0) (IEEE division, then
// round-to-nearest-even with saturation).  The layout of the work is new: the
// reference stages a 128x128 fp32 block in a 64 KB static shared array, which
// does not even assemble (static shared memory is limited to 48 KB); here the
// block lives in registers and the scales are written coalesced.
#include <cuda_fp8.h>

#include "host_common.h"
#include "sm100.cuh"

namespace llmmm {

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  }
  return v;
}

__device__ __forceinline__ float amax4(float4 v)
{
  return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

// x / s, correctly rounded, for |x| <= 448 s: with r = RN(1/s) and q = RN(x r), one residual step
// RN(q + r * (x - s q)) gives the correctly rounded quotient (Markstein) as long as nothing underflows; where
// it could (|x/s| below the normal range) the e4m3 result is zero either way.  Three instructions per element
// instead of the division sequence, which cost a third of this kernel's issue slots.
__device__ __forceinline__ float div_by_scale(float x, float s, float r)
{
  const float q = __fmul_rn(x, r);
  const float e = __fmaf_rn(-s, q, x);
  return __fmaf_rn(e, r, q);
}

__device__ __forceinline__ uint32_t quant4(float4 v, float s)
{
  float a, b, c, d;
  if (s >= 1e-30f) {
    const float r = __frcp_rn(s);
    a = div_by_scale(v.x, s, r);
    b = div_by_scale(v.y, s, r);
    c = div_by_scale(v.z, s, r);
    d = div_by_scale(v.w, s, r);
  }
  else {
    // scales this small (the reciprocal would overflow) and the all-zero group take the plain division
    a = s != 0.0f ? __fdiv_rn(v.x, s) : 0.0f;
    b = s != 0.0f ? __fdiv_rn(v.y, s) : 0.0f;
    c = s != 0.0f ? __fdiv_rn(v.z, s) : 0.0f;
    d = s != 0.0f ? __fdiv_rn(v.w, s) : 0.0f;
  }
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// One warp quantises Q1_ROWS consecutive rows of one 128-wide K group: per row
// the 32 lanes hold one float4 each (a coalesced 512-byte read, all rows' loads in
// flight together), the row amax is a warp reduction, and lane r keeps the scale
// of row r so that the scales leave as one 32-byte sector of scale[(K/128), M].
constexpr int Q1_ROWS  = 8;
constexpr int Q1_WARPS = 8;

__global__ void __launch_bounds__(Q1_WARPS * 32)
  quant_1x128_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, int M, int K)
{
  pdl_launch_dependents();  // see sm100.cuh: the next kernel may start its set-up, this one waits for its predecessor
  pdl_wait();
  const int lane    = threadIdx.x & 31;
  const int warp    = threadIdx.x >> 5;
  const int groups  = K / 128;
  const long long w = (long long)blockIdx.x * Q1_WARPS + warp;
  const int row_blocks = (M + Q1_ROWS - 1) / Q1_ROWS;
  if (w >= (long long)row_blocks * groups) {
    return;
  }
  // consecutive warps walk along K first so that a CTA reads long row segments
  const int g  = (int)(w % groups);
  const int m0 = (int)(w / groups) * Q1_ROWS;

  float my_scale = 0.0f;
#pragma unroll 1
  for (int r0 = 0; r0 < Q1_ROWS; r0 += 8) {
    float4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int m = m0 + r0 + j;
      v[j]        = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < M) {
        v[j] = __ldcs(reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)g * 128) + lane);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int   m    = m0 + r0 + j;
      const float amax = warp_max(amax4(v[j]));
      const float s    = __fdiv_rn(amax, 448.0f);
      if (lane == r0 + j) {
        my_scale = s;
      }
      if (m < M) {
        reinterpret_cast<uint32_t*>(q + (size_t)m * K + (size_t)g * 128)[lane] = quant4(v[j], s);
      }
    }
  }
  if (lane < Q1_ROWS && m0 + lane < M) {
    scale[(size_t)g * M + m0 + lane] = my_scale;
  }
}

// One CTA of 256 threads quantises one 128x128 block held in registers
// (16 float4 per thread): block amax by warp shuffles and an 8-entry shared
// array, then the conversion straight from registers.
__global__ void __launch_bounds__(256)
  quant_128x128_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, int rows, int cols)
{
  __shared__ float warp_amax[8];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int cb   = blockIdx.x;
  const int rb   = blockIdx.y;
  const int CB   = cols / 128;

  float4 v[16];
  float  amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int r = rb * 128 + j * 8 + warp;
    v[j]        = __ldcs(reinterpret_cast<const float4*>(x + (size_t)r * cols + (size_t)cb * 128) + lane);
    amax        = fmaxf(amax, amax4(v[j]));
  }
  amax = warp_max(amax);
  if (lane == 0) {
    warp_amax[warp] = amax;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    amax = fmaxf(amax, warp_amax[i]);
  }
  const float s = __fdiv_rn(amax, 448.0f);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int r = rb * 128 + j * 8 + warp;
    reinterpret_cast<uint32_t*>(q + (size_t)r * cols + (size_t)cb * 128)[lane] = quant4(v[j], s);
  }
  if (threadIdx.x == 0) {
    scale[(size_t)rb * CB + cb] = s;
  }
}

// RMSNorm fused in front of the activation quantiser: y = x * rsqrt(mean(x^2) + eps) * weight, then the 1x128
// quantisation of y.  One CTA per row: it sums the squares, then scales and quantises one 128-wide group per
// warp at a time.  A row of up to 8192 values is kept in registers in between (one pass over memory); a longer
// one is re-read from L2.
constexpr int RN_THREADS = 256;

// RESIDENT: float4 values of the row a thread keeps (0: none, the row is re-read from L2 for the second phase).
template<int RESIDENT>
__global__ void __launch_bounds__(RN_THREADS)
  rmsnorm_quant_1x128_kernel(const float* __restrict__ x, const float* __restrict__ weight, float eps, uint8_t* __restrict__ q,
                             float* __restrict__ scale, int M, int K)
{
  __shared__ float warp_sum[RN_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int     lane = threadIdx.x & 31;
  const int     warp = threadIdx.x >> 5;
  const int     m    = blockIdx.x;
  const float4* row  = reinterpret_cast<const float4*>(x + (size_t)m * K);
  // Rows of up to 8192 values stay in registers between the two phases (RESIDENT float4 per thread): element
  // threadIdx.x + 256 j of the row, as float4, is lane `lane` of the 128-wide group warp + 8 j, so the thread
  // that read a value for the sum of squares is the one that quantises it, and x is read from memory once.
  constexpr bool resident = RESIDENT > 0;
  float4         v[resident ? RESIDENT : 1];
  float          ss = 0.0f;
  if constexpr (resident) {
#pragma unroll
    for (int j = 0; j < RESIDENT; ++j) {
      const int i = threadIdx.x + j * RN_THREADS;
      v[j]        = i < K / 4 ? __ldg(row + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int j = 0; j < RESIDENT; ++j) {  // (zeros beyond the row add nothing: same sum, same order as below)
      ss = fmaf(v[j].x, v[j].x, ss);
      ss = fmaf(v[j].y, v[j].y, ss);
      ss = fmaf(v[j].z, v[j].z, ss);
      ss = fmaf(v[j].w, v[j].w, ss);
    }
  }
  else {
    for (int i = threadIdx.x; i < K / 4; i += RN_THREADS) {
      const float4 t = __ldg(row + i);
      ss             = fmaf(t.x, t.x, ss);
      ss             = fmaf(t.y, t.y, ss);
      ss             = fmaf(t.z, t.z, ss);
      ss             = fmaf(t.w, t.w, ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  }
  if (lane == 0) {
    warp_sum[warp] = ss;
  }
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < RN_THREADS / 32; ++i) {
    total += warp_sum[i];  // the same order in every thread
  }
  const float inv = __frsqrt_rn(__fdiv_rn(total, (float)K) + eps);
  const float4* wrow = reinterpret_cast<const float4*>(weight);
  auto emit = [&](int g, const float4& t) {
    const float4 w = __ldg(wrow + g * 32 + lane);
    float4       y;
    y.x = __fmul_rn(__fmul_rn(t.x, inv), w.x);
    y.y = __fmul_rn(__fmul_rn(t.y, inv), w.y);
    y.z = __fmul_rn(__fmul_rn(t.z, inv), w.z);
    y.w = __fmul_rn(__fmul_rn(t.w, inv), w.w);
    const float amax = warp_max(amax4(y));
    const float sc   = __fdiv_rn(amax, 448.0f);
    reinterpret_cast<uint32_t*>(q + (size_t)m * K + (size_t)g * 128)[lane] = quant4(y, sc);
    if (lane == 0) {
      scale[(size_t)g * M + m] = sc;
    }
  };
  if constexpr (resident) {
#pragma unroll
    for (int j = 0; j < RESIDENT; ++j) {
      const int g = warp + j * (RN_THREADS / 32);
      if (g < K / 128) {
        emit(g, v[j]);
      }
    }
  }
  else {
    for (int g = warp; g < K / 128; g += RN_THREADS / 32) {
      emit(g, __ldg(row + g * 32 + lane));  // second pass: from L2
    }
  }
}

// h = silu(gate) * up for one row and one 128-wide group per warp, then the output quantisation rule of the
// GEMM epilogue (scale = amax / 448, q = e4m3(h * (448 / amax))): the same arithmetic as the fused epilogue of
// the prefill-sized kernel, applied to an accumulator that a decode-sized GEMM left in scratch.
__global__ void __launch_bounds__(256)
  swiglu_quant_1x128_kernel(const float* __restrict__ acc, uint8_t* __restrict__ H, float* __restrict__ H_s, int M, int I)
{
  pdl_launch_dependents();
  pdl_wait();
  const int lane   = threadIdx.x & 31;
  const int groups = I / 128;
  const int w      = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= M * groups) {
    return;
  }
  const int    m = w / groups, g = w % groups;
  const float* row = acc + (size_t)m * 2 * I;
  const float4 ga  = __ldcs(reinterpret_cast<const float4*>(row + (size_t)g * 128) + lane);
  const float4 up  = __ldcs(reinterpret_cast<const float4*>(row + I + (size_t)g * 128) + lane);
  float4       h;
  h.x = __fdividef(ga.x, 1.0f + __expf(-ga.x)) * up.x;
  h.y = __fdividef(ga.y, 1.0f + __expf(-ga.y)) * up.y;
  h.z = __fdividef(ga.z, 1.0f + __expf(-ga.z)) * up.z;
  h.w = __fdividef(ga.w, 1.0f + __expf(-ga.w)) * up.w;
  const float amax  = warp_max(amax4(h));
  const float scale = __fdiv_rn(amax, 448.0f);
  const float inv   = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(h.x * inv, h.y * inv), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(h.z * inv, h.w * inv), __NV_SATFINITE, __NV_E4M3);
  reinterpret_cast<uint32_t*>(H + (size_t)m * I + (size_t)g * 128)[lane] = lo | (hi << 16);
  if (lane == 0) {
    H_s[(size_t)g * M + m] = scale;
  }
}

int launch_swiglu_quant(const float* acc, void* H, float* H_s, int M, int I, cudaStream_t stream)
{
  const int warps = M * (I / 128);
  LLMMM_CUDA_TRY(launch_pdl(swiglu_quant_1x128_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, stream, 1, acc,
                            static_cast<uint8_t*>(H), H_s, M, I));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

// The qkv hook (per-head RMSNorm of query / key heads, rotary embedding, 1x128 quantisation) applied to an fp32
// accumulator [M, N] that a decode-sized GEMM left in scratch: one warp per (row, head); lane l holds columns
// 2l, 2l+1 and 64+2l, 64+2l+1, i.e. two rotation pairs.  Same arithmetic as the fused epilogue of the
// prefill-sized kernel up to the order of the sum of squares.
__global__ void __launch_bounds__(256)
  rope_quant_1x128_kernel(const float* __restrict__ acc, uint8_t* __restrict__ C, float* __restrict__ C_s,
                          const __grid_constant__ RopeHook hook, int M, int N, uint32_t* status)
{
  pdl_launch_dependents();
  pdl_wait();
  const int lane  = threadIdx.x & 31;
  const int heads = N / 128;
  const int w     = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= M * heads) {
    return;
  }
  const int    m = w / heads, h = w % heads;
  const float* row = acc + (size_t)m * N + (size_t)h * 128;
  float2       lo  = __ldcs(reinterpret_cast<const float2*>(row) + lane);
  float2       hi  = __ldcs(reinterpret_cast<const float2*>(row + 64) + lane);
  const int    kind = h < hook.n_q ? 0 : (h < hook.n_q + hook.n_kv ? 1 : 2);
  if (kind < 2) {
    const float* wgt = kind == 0 ? hook.q_w : hook.k_w;
    if (wgt != nullptr) {
      float ss = fmaf(lo.x, lo.x, fmaf(lo.y, lo.y, fmaf(hi.x, hi.x, hi.y * hi.y)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
      }
      const float  inv = __frcp_rn(__fsqrt_rn(fmaf(ss, 1.0f / 128.0f, hook.eps)));
      const float2 wl  = __ldg(reinterpret_cast<const float2*>(wgt) + lane);
      const float2 wh  = __ldg(reinterpret_cast<const float2*>(wgt + 64) + lane);
      lo.x = lo.x * inv * wl.x;
      lo.y = lo.y * inv * wl.y;
      hi.x = hi.x * inv * wh.x;
      hi.y = hi.y * inv * wh.y;
    }
    const int p_raw = __ldg(hook.pos + m);
    const int p_row = min(max(p_raw, 0), hook.rows - 1);
    if (p_row != p_raw && lane == 0) {
      atomicCAS(status, 0u, (uint32_t)DEV_BAD_POSITION);  // the access outside the tables is not made
    }
    const size_t p = (size_t)p_row * 64;
    const float2 c = __ldg(reinterpret_cast<const float2*>(hook.cos + p) + lane);
    const float2 s = __ldg(reinterpret_cast<const float2*>(hook.sin + p) + lane);
    const float2 l0 = lo, h0 = hi;
    lo.x = __fmaf_rn(l0.x, c.x, -__fmul_rn(h0.x, s.x));
    lo.y = __fmaf_rn(l0.y, c.y, -__fmul_rn(h0.y, s.y));
    hi.x = __fmaf_rn(h0.x, c.x, __fmul_rn(l0.x, s.x));
    hi.y = __fmaf_rn(h0.y, c.y, __fmul_rn(l0.y, s.y));
  }
  const float amax  = warp_max(fmaxf(fmaxf(fabsf(lo.x), fabsf(lo.y)), fmaxf(fabsf(hi.x), fabsf(hi.y))));
  const float scale = __fdiv_rn(amax, 448.0f);
  const float inv   = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
  uint8_t*    dst   = C + (size_t)m * N + (size_t)h * 128;
  reinterpret_cast<uint16_t*>(dst)[lane] =
    (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(lo.x * inv, lo.y * inv), __NV_SATFINITE, __NV_E4M3);
  reinterpret_cast<uint16_t*>(dst + 64)[lane] =
    (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(hi.x * inv, hi.y * inv), __NV_SATFINITE, __NV_E4M3);
  if (lane == 0) {
    C_s[(size_t)h * M + m] = scale;
  }
}

int launch_rope_quant(const float* acc, void* C, float* C_s, const RopeHook& hook, int M, int N, uint32_t* status,
                      cudaStream_t stream)
{
  const int warps = M * (N / 128);
  LLMMM_CUDA_TRY(launch_pdl(rope_quant_1x128_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, stream, 1, acc,
                            static_cast<uint8_t*>(C), C_s, hook, M, N, status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

}  // namespace llmmm

extern "C" {

int llmmm_fp8_rmsnorm_quant_1x128(const float* x, const float* weight, float eps, void* q, float* scale, int M, int K,
                                  llmmm_stream_t stream)
{
  using namespace llmmm;
  if (x == nullptr || weight == nullptr || q == nullptr || scale == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (M < 1 || K < 128 || (K % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "M or K are not aligned. (need M>=1, K%%128==0; got %d %d)", M, K);
  }
  if (((uintptr_t)x | (uintptr_t)q | (uintptr_t)weight) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "x, weight and q must be 16-byte aligned");
  }
  if (!(eps >= 0.0f)) {
    return set_error(LLMMM_ERR_SHAPE, "eps must be non-negative");
  }
  if (device_info() == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  // as few resident values as the row needs: registers decide how many rows an SM works on at a time
  auto* kernel = K <= 2 * RN_THREADS * 4 ? rmsnorm_quant_1x128_kernel<2>
               : K <= 4 * RN_THREADS * 4 ? rmsnorm_quant_1x128_kernel<4>
               : K <= 8 * RN_THREADS * 4 ? rmsnorm_quant_1x128_kernel<8> : rmsnorm_quant_1x128_kernel<0>;
  LLMMM_CUDA_TRY(launch_pdl(kernel, dim3((unsigned)M), dim3(RN_THREADS), 0,
                            reinterpret_cast<cudaStream_t>(stream), 1, x, weight, eps, static_cast<uint8_t*>(q), scale, M, K));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

int llmmm_fp8_quant_1x128(const float* x, void* q, float* scale, int M, int K, llmmm_stream_t stream)
{
  using namespace llmmm;
  if (x == nullptr || q == nullptr || scale == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (M < 1 || K < 128 || (K % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "M or K are not aligned. (need M>=1, K%%128==0; got %d %d)", M, K);
  }
  if (((uintptr_t)x | (uintptr_t)q) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "x and q must be 16-byte aligned");
  }
  if (device_info() == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  const long long warps  = (long long)((M + Q1_ROWS - 1) / Q1_ROWS) * (K / 128);
  const long long blocks = (warps + Q1_WARPS - 1) / Q1_WARPS;
  LLMMM_CUDA_TRY(launch_pdl(quant_1x128_kernel, dim3((unsigned)blocks), dim3(Q1_WARPS * 32), 0,
                            reinterpret_cast<cudaStream_t>(stream), 1, x, static_cast<uint8_t*>(q), scale, M, K));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

int llmmm_fp8_quant_128x128(const float* x, void* q, float* scale, int rows, int cols, llmmm_stream_t stream)
{
  using namespace llmmm;
  if (x == nullptr || q == nullptr || scale == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (rows < 128 || cols < 128 || (rows % 128) != 0 || (cols % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "rows or cols are not aligned. (need multiples of 128; got %d %d)", rows, cols);
  }
  if (((uintptr_t)x | (uintptr_t)q) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "x and q must be 16-byte aligned");
  }
  if (device_info() == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  dim3 grid(cols / 128, rows / 128);
  LLMMM_CUDA_TRY(launch_pdl(quant_128x128_kernel, grid, dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 1, x,
                            static_cast<uint8_t*>(q), scale, rows, cols));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

}  // extern "C"
