// FP8 e4m3 blockwise-quantised GEMM for sm_100a with the output's 1x128
// re-quantisation fused into the epilogue.
//
//   acc[m,n] = sum_kb ( sum_{k in kb} A_q[m,k] * B_q[n,k] ) * ( A_s[kb,m] * B_s[n/128,kb] )
//   C_s[n/128, m] = amax_{n in group} |acc| / 448,   C_q = e4m3( acc * 448/amax )
//
// Replaces the reference's mma.sync.m16n8k32 kernel family
// (examples/005.fp8.mm.cu:565-2464, launchers :2466-2577; fp32-output form
// :51-246).  The arithmetic contract kept from it: the scale product
// A_s*B_s is rounded to fp32 first (:1066-1067), each 128-K block is summed by
// the tensor core from zero and added with one FMA (:890-901), and C is
// quantised with scale = amax/448, q = e4m3(acc * (448/amax)) (:1111-1137).
//
// Structure (nothing of the reference's is kept):
//   * persistent grid, one CTA per SM, 128x256 output tiles (two 1x128 scale
//     groups per row);
//   * warp 0 streams A_q (128x128 B) and B_q (256x128 B) K-blocks with TMA into
//     a 4-stage ring of 128-byte-swizzled tiles;
//   * warp 1 issues, per K-block, four tcgen05.mma.kind::f8f6f4 (128x256x32)
//     that start from zero into one of two 256-column TMEM "partial" stages;
//   * warps 4-11 (two warpgroups, 256 threads, given most of the register file
//     with setmaxnreg) promote: each thread owns one output row and one
//     128-column scale group, reads the finished partial with tcgen05.ld (the
//     next 32 columns are in flight while the current 32 are accumulated) and
//     does acc = fma(partial, A_s*B_s, acc) in registers while the tensor core
//     fills the other partial stage; the scale product of the next K-block is
//     fetched one block ahead;
//   * after the last K-block the same threads reduce their 128 values to the
//     group absmax (thread-local: no shuffles in this orientation), convert to
//     e4m3 and store one 128-byte line each, plus the coalesced scale column.
#include <cuda_fp8.h>

#include "host_common.h"
#include "sm100.cuh"

namespace llmmm {

namespace fp8cfg {
constexpr int      BM         = 128;
constexpr int      BN         = 256;
constexpr int      BK         = 128;  // one scale block of K = one 128-byte swizzle row
constexpr int      UMMA_K     = 32;
constexpr int      STAGES     = 4;
constexpr int      PROMO_WARPS = 8;
constexpr int      THREADS    = 128 + PROMO_WARPS * 32;  // warpgroup 0: TMA / MMA; warpgroups 1-2: promotion
constexpr int      REGS_CTRL  = 40;                      // register budget after setmaxnreg: control warpgroup
constexpr int      REGS_PROMO = 232;                     //   and promotion warpgroups (128*40 + 256*232 = 384*168)
constexpr uint32_t A_BYTES    = BM * BK;
constexpr uint32_t B_BYTES    = BN * BK;
constexpr uint32_t STAGE_TX   = A_BYTES + B_BYTES;
constexpr uint32_t OFF_A      = 0;
constexpr uint32_t OFF_B      = OFF_A + STAGES * A_BYTES;
constexpr uint32_t OFF_BAR    = OFF_B + STAGES * B_BYTES;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr uint32_t TMEM_COLS  = 512;  // two partial stages of 256 columns
}  // namespace fp8cfg

struct Fp8Bars {
  uint64_t full[fp8cfg::STAGES];
  uint64_t empty[fp8cfg::STAGES];
  uint64_t part_full[2];
  uint64_t part_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template<int REGS>
__device__ __forceinline__ void setmaxnreg_inc()
{
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}

template<int REGS>
__device__ __forceinline__ void setmaxnreg_dec()
{
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d)
{
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// OUT_F32 = false: C_q e4m3 + C_s;  true: C fp32, no quantisation.
template<bool OUT_F32>
__global__ void __launch_bounds__(fp8cfg::THREADS, 1) fp8_blockwise_gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                                                const __grid_constant__ CUtensorMap tm_b,
                                                                                const float* __restrict__ A_s,
                                                                                const float* __restrict__ B_s,
                                                                                void* __restrict__ C_out,
                                                                                float* __restrict__ C_s,
                                                                                int       M,
                                                                                int       N,
                                                                                int       K,
                                                                                uint32_t* status)
{
  using namespace fp8cfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Fp8Bars* bars = reinterpret_cast<Fp8Bars*>(smem + OFF_BAR);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles   = (M + BM - 1) / BM;
  const int n_tiles   = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks  = K / BK;
  const int n_groups  = N / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int p = 0; p < 2; ++p) {
      mbar_init(&bars->part_full[p], 1);
      mbar_init(&bars->part_empty[p], PROMO_WARPS);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc<TMEM_COLS>(&bars->tmem_base);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp < 4) {
    setmaxnreg_dec<REGS_CTRL>();
  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM;
        const int n0 = (tile / m_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s  = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          mbar_wait(&bars->empty[s], ph ^ 1, DEV_WAIT_SMEM_EMPTY, abort_flag, status);
          mbar_arrive_expect_tx(&bars->full[s], STAGE_TX);
          tma_load_2d(smem + OFF_A + s * A_BYTES, &tm_a, &bars->full[s], kb * BK, m0);
          tma_load_2d(smem + OFF_B + s * B_BYTES, &tm_b, &bars->full[s], kb * BK, n0);
        }
      }
    }
  }
  else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*e4m3*/ 0, 0, 0, 0, BM, BN);
      uint32_t           it    = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s  = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const uint32_t p  = it & 1;
          const uint32_t pp = (it >> 1) & 1;
          mbar_wait(&bars->part_empty[p], pp ^ 1, DEV_WAIT_TMEM_EMPTY, abort_flag, status);
          mbar_wait(&bars->full[s], ph, DEV_WAIT_SMEM_FULL, abort_flag, status);
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(smem_u32(smem + OFF_A + s * A_BYTES), 0, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_u32(smem + OFF_B + s * B_BYTES), 0, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            tc_mma_f8(tmem_base + p * BN, da + (uint64_t)((kk * UMMA_K) >> 4), db + (uint64_t)((kk * UMMA_K) >> 4), idesc, kk != 0);
          }
          tc_commit(&bars->empty[s]);
          tc_commit(&bars->part_full[p]);
        }
      }
    }
  }
  }
  else {
    setmaxnreg_inc<REGS_PROMO>();
    // ------------------------------------------- promotion + epilogue ----
    const int      quarter = warp & 3;         // TMEM lane quarter this warp may read
    const int      half    = (warp - 4) >> 2;  // which 128-column scale group of the tile
    const uint32_t t_lane  = ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 128);
    uint32_t       it      = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int  m    = (tile % m_tiles) * BM + quarter * 32 + lane;
      const int  ng   = (tile / m_tiles) * (BN / 128) + half;  // global 128-column group
      const bool m_ok = m < M;
      const bool g_ok = ng < n_groups;
      const float* a_s = A_s + (m_ok ? m : 0);
      const float* b_s = B_s + (size_t)(g_ok ? ng : 0) * k_blocks;

      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) {
        acc[i] = 0.0f;
      }

      // Scale operands are fetched PREFETCH K-blocks ahead of their use: under the TMA load traffic
      // an L2 hit takes longer than one K-block lasts.  The empty asm pins the first use of a
      // fetched value to the top of its own iteration, so the wait for it is never moved up to
      // the load.
      constexpr int PREFETCH = 4;
      float         a_pf[PREFETCH], b_pf[PREFETCH];
#pragma unroll
      for (int j = 0; j < PREFETCH; ++j) {
        a_pf[j] = (j < k_blocks) ? __ldg(a_s + (size_t)j * M) : 0.0f;
        b_pf[j] = (j < k_blocks) ? __ldg(b_s + j) : 0.0f;
      }
      for (int kb0 = 0; kb0 < k_blocks; kb0 += PREFETCH) {
#pragma unroll
      for (int j = 0; j < PREFETCH; ++j) {
        const int kb = kb0 + j;
        if (kb >= k_blocks) {
          break;
        }
        const uint32_t p  = it & 1;
        const uint32_t pp = (it >> 1) & 1;
        float a_cur = a_pf[j], b_cur = b_pf[j];
        asm volatile("" : "+f"(a_cur), "+f"(b_cur));
        // one fp32 rounding of the scale product, as in the reference
        const float sc = __fmul_rn(a_cur, b_cur);
        if (kb + PREFETCH < k_blocks) {
          a_pf[j] = __ldg(a_s + (size_t)(kb + PREFETCH) * M);
          b_pf[j] = __ldg(b_s + kb + PREFETCH);
        }
        mbar_wait(&bars->part_full[p], pp, DEV_WAIT_TMEM_FULL, abort_flag, status);
        tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + p * BN + t_lane;
        uint32_t       v0[32], v1[32];
        tmem_ld_32x32b_x32(t_addr, v0);
        tmem_ld_wait();
        tmem_ld_32x32b_x32(t_addr + 32, v1);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = __fmaf_rn(__uint_as_float(v0[i]), sc, acc[i]);
        }
        tmem_ld_wait();
        tmem_ld_32x32b_x32(t_addr + 64, v0);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[32 + i] = __fmaf_rn(__uint_as_float(v1[i]), sc, acc[32 + i]);
        }
        tmem_ld_wait();
        tmem_ld_32x32b_x32(t_addr + 96, v1);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[64 + i] = __fmaf_rn(__uint_as_float(v0[i]), sc, acc[64 + i]);
        }
        tmem_ld_wait();
        // every column of this thread's part of the partial stage has been read
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->part_empty[p]);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[96 + i] = __fmaf_rn(__uint_as_float(v1[i]), sc, acc[96 + i]);
        }
        ++it;
      }
      }

      if (m_ok && g_ok) {
        if constexpr (OUT_F32) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(C_out) + (size_t)m * N + (size_t)ng * 128);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
          }
        }
        else {
          float amax = 0.0f;
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            amax = fmaxf(amax, fabsf(acc[i]));
          }
          const float scale     = __fdiv_rn(amax, 448.0f);
          const float scale_inv = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(C_out) + (size_t)m * N + (size_t)ng * 128);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint4 q;
            q.x    = pack_e4m3x4(acc[16 * i + 0] * scale_inv, acc[16 * i + 1] * scale_inv, acc[16 * i + 2] * scale_inv, acc[16 * i + 3] * scale_inv);
            q.y    = pack_e4m3x4(acc[16 * i + 4] * scale_inv, acc[16 * i + 5] * scale_inv, acc[16 * i + 6] * scale_inv, acc[16 * i + 7] * scale_inv);
            q.z    = pack_e4m3x4(acc[16 * i + 8] * scale_inv, acc[16 * i + 9] * scale_inv, acc[16 * i + 10] * scale_inv, acc[16 * i + 11] * scale_inv);
            q.w    = pack_e4m3x4(acc[16 * i + 12] * scale_inv, acc[16 * i + 13] * scale_inv, acc[16 * i + 14] * scale_inv, acc[16 * i + 15] * scale_inv);
            dst[i] = q;
          }
          C_s[(size_t)ng * M + m] = scale;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

template<bool OUT_F32>
static int launch_fp8(const void*  A,
                      const float* A_s,
                      const void*  B,
                      const float* B_s,
                      void*        C,
                      float*       C_s,
                      int          M,
                      int          N,
                      int          K,
                      cudaStream_t stream)
{
  using namespace fp8cfg;
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  CUtensorMap tm_a, tm_b;
  if (!make_tmap_2d(&tm_a, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_b, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(cudaFuncSetAttribute(
      fp8_blockwise_gemm_kernel<OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    attr_set[info->device] = true;
  }
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = (N + BN - 1) / BN;
  const int tiles   = m_tiles * n_tiles;
  const int grid    = tiles < info->sm_count ? tiles : info->sm_count;
  fp8_blockwise_gemm_kernel<OUT_F32>
    <<<grid, THREADS, SMEM_BYTES, stream>>>(tm_a, tm_b, A_s, B_s, C, C_s, M, N, K, info->status);
  g_launches.fetch_add(1);
  LLMMM_CUDA_TRY(cudaGetLastError());
  return LLMMM_OK;
}

static int check_fp8_args(const void* A, const void* A_s, const void* B, const void* B_s, const void* C, int M, int N, int K)
{
  if (A == nullptr || A_s == nullptr || B == nullptr || B_s == nullptr || C == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (M < 1 || N < 128 || K < 128 || (N % 128) != 0 || (K % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "M or N or K are not aligned. (need M>=1, N%%128==0, K%%128==0; got %d %d %d)", M, N, K);
  }
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "A, B and C must be 16-byte aligned");
  }
  return LLMMM_OK;
}

}  // namespace llmmm

extern "C" {

int llmmm_fp8_blockwise_mm_e4m3out(const void*    A,
                                   const float*   A_scale_t,
                                   const void*    B_t,
                                   const float*   B_scale_t,
                                   void*          C,
                                   float*         C_scale_t,
                                   int            M,
                                   int            N,
                                   int            K,
                                   llmmm_stream_t stream)
{
  int rc = llmmm::check_fp8_args(A, A_scale_t, B_t, B_scale_t, C, M, N, K);
  if (rc != LLMMM_OK) {
    return rc;
  }
  if (C_scale_t == nullptr) {
    return llmmm::set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  rc             = llmmm::launch_decode(false, A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K, s);
  if (rc >= 0) {
    return rc;
  }
  return llmmm::launch_fp8<false>(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K, s);
}

int llmmm_fp8_blockwise_mm_f32out(const void*    A,
                                  const float*   A_scale_t,
                                  const void*    B_t,
                                  const float*   B_scale_t,
                                  float*         C,
                                  int            M,
                                  int            N,
                                  int            K,
                                  llmmm_stream_t stream)
{
  int rc = llmmm::check_fp8_args(A, A_scale_t, B_t, B_scale_t, C, M, N, K);
  if (rc != LLMMM_OK) {
    return rc;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  rc             = llmmm::launch_decode(true, A, A_scale_t, B_t, B_scale_t, C, nullptr, M, N, K, s);
  if (rc >= 0) {
    return rc;
  }
  return llmmm::launch_fp8<true>(A, A_scale_t, B_t, B_scale_t, C, nullptr, M, N, K, s);
}

}  // extern "C"
