// FP16 / BF16 GEMM for sm_100a:  C[M,N] = A[M,K] * B[K,N], row-major, fp32
// accumulation in tensor memory, one round-to-nearest conversion of the result.
//
// Replaces the reference's LLMMM::fp16_mm<T> (launcher src/mm/fp16/mm.cu:7-42,
// kernel src/mm/fp16/mm.cuh:10-684, an mma.sync.m16n8k16 + ldmatrix kernel with
// a 256x256 CTA tile).  Nothing of that kernel's structure is kept:
//
//   * persistent grid, one CTA per SM, static round-robin over 128x256 tiles;
//   * warp 0 (one lane) streams A (K-major) and B (N-major, read in place from
//     the row-major [K,N] array: no transpose pass) with TMA into a 4-stage
//     ring of 128-byte-swizzled shared-memory tiles, completion on mbarriers;
//   * warp 1 (one lane) issues tcgen05.mma.kind::f16 (128x256x16) into one of
//     two 256-column TMEM accumulators and commits ring slots back to the
//     producer and finished accumulators to the epilogue;
//   * warps 4-7 drain an accumulator with tcgen05.ld (each lane owns one
//     output row), convert to the 16-bit type, stage 32x64 sub-tiles in
//     swizzled shared memory and write them with TMA stores, while the MMA warp
//     already fills the other accumulator with the next tile.
//
// Edge tiles rely on TMA: out-of-range loads read zeros, stores are clipped.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <type_traits>

#include "host_common.h"
#include "pair_walk.cuh"
#include "sm100.cuh"

namespace llmmm {

namespace fp16cfg {
constexpr int      BM          = 128;
constexpr int      BN          = 256;
constexpr int      BK          = 64;  // 64 x 2 B = one 128-byte swizzle row of A
constexpr int      UMMA_K      = 16;
constexpr int      STAGES      = 4;
constexpr int      THREADS     = 256;
constexpr uint32_t A_BYTES     = BM * BK * 2;         // 16 KB
constexpr uint32_t B_BOX_BYTES = 64 * BK * 2;         // one 64(n) x 64(k) box: 8 KB
constexpr uint32_t B_BYTES     = B_BOX_BYTES * (BN / 64);  // 32 KB
constexpr uint32_t STAGE_TX    = A_BYTES + B_BYTES;
constexpr uint32_t C_WARP_BUF  = 32 * 128;  // 32 rows x 64 halves
constexpr uint32_t OFF_A       = 0;
constexpr uint32_t OFF_B       = OFF_A + STAGES * A_BYTES;
constexpr uint32_t OFF_C       = OFF_B + STAGES * B_BYTES;
constexpr uint32_t OFF_BAR     = OFF_C + 4 * 2 * C_WARP_BUF;
constexpr uint32_t SMEM_BYTES  = OFF_BAR + 256 + 1024;  // + barrier block + alignment slack
constexpr uint32_t TMEM_COLS   = 512;                   // two 256-column accumulators
}  // namespace fp16cfg

struct Fp16Bars {
  uint64_t full[fp16cfg::STAGES];
  uint64_t empty[fp16cfg::STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template<typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);

template<>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b)
{
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template<>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b)
{
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template<typename T>
__global__ void __launch_bounds__(fp16cfg::THREADS, 1) fp16_gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                                        const __grid_constant__ CUtensorMap tm_b,
                                                                        const __grid_constant__ CUtensorMap tm_c,
                                                                        int                                 M,
                                                                        int                                 N,
                                                                        int                                 K,
                                                                        uint32_t*                           status)
{
  using namespace fp16cfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t*  smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Fp16Bars* bars = reinterpret_cast<Fp16Bars*>(smem + OFF_BAR);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles   = (M + BM - 1) / BM;
  const int n_tiles   = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_iters   = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 4);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b);
    prefetch_tmap(&tm_c);
  }
  if (warp == 2) {
    tmem_alloc<TMEM_COLS>(&bars->tmem_base);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // no global memory touched so far: this may overlap the tail of the previous kernel on the stream
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM;
        const int n0 = (tile / m_tiles) * BN;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const uint32_t s  = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          mbar_wait(&bars->empty[s], ph ^ 1, DEV_WAIT_SMEM_EMPTY, abort_flag, status);
          mbar_arrive_expect_tx(&bars->full[s], STAGE_TX);
          tma_load_2d(smem + OFF_A + s * A_BYTES, &tm_a, &bars->full[s], kb * BK, m0);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) {
            tma_load_2d(smem + OFF_B + s * B_BYTES + j * B_BOX_BYTES, &tm_b, &bars->full[s], n0 + j * 64, kb * BK);
          }
        }
      }
    }
  }
  else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t kFmt  = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(kFmt, kFmt, /*a_mn=*/0, /*b_mn=*/1, BM, BN);
      uint32_t           it    = 0;
      uint32_t           t     = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
        const uint32_t acc    = t & 1;
        const uint32_t acc_ph = (t >> 1) & 1;
        mbar_wait(&bars->tmem_empty[acc], acc_ph ^ 1, DEV_WAIT_TMEM_EMPTY, abort_flag, status);
        tc_fence_after_sync();
        const uint32_t d_addr = tmem_base + acc * BN;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const uint32_t s  = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          mbar_wait(&bars->full[s], ph, DEV_WAIT_SMEM_FULL, abort_flag, status);
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(smem_u32(smem + OFF_A + s * A_BYTES), 0, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_u32(smem + OFF_B + s * B_BYTES), B_BOX_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // A: 16 k-elements = 32 B inside the swizzled row; B: 16 k-rows of 128 B.
            tc_mma_f16(d_addr,
                       da + (uint64_t)((kk * UMMA_K * 2) >> 4),
                       db + (uint64_t)((kk * UMMA_K * 128) >> 4),
                       idesc,
                       (kb | kk) != 0);
          }
          tc_commit(&bars->empty[s]);
        }
        tc_commit(&bars->tmem_full[acc]);
      }
    }
  }
  else if (warp >= 4) {
    // ---------------------------------------------------------- epilogue --
    const int      ew       = warp - 4;  // == warp % 4: the TMEM lane quarter this warp may read
    uint8_t*       cbuf     = smem + OFF_C + ew * 2 * C_WARP_BUF;
    uint32_t       t        = 0;
    uint32_t       chunk_it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      const int      m0     = (tile % m_tiles) * BM;
      const int      n0     = (tile / m_tiles) * BN;
      const uint32_t acc    = t & 1;
      const uint32_t acc_ph = (t >> 1) & 1;
      mbar_wait(&bars->tmem_full[acc], acc_ph, DEV_WAIT_TMEM_FULL, abort_flag, status);
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(ew * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c, ++chunk_it) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_addr + c * 64, v0);
        tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
        tmem_ld_wait();
        if (c == BN / 64 - 1) {
          // the accumulator is drained: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&bars->tmem_empty[acc]);
          }
        }
        uint8_t* buf = cbuf + (chunk_it & 1) * C_WARP_BUF;
        // the TMA store issued from this buffer two chunks ago must have read it
        if (lane == 0) {
          tma_store_wait_read<1>();
        }
        __syncwarp();
        uint8_t* row = buf + lane * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 q;
          q.x = pack2<T>(__uint_as_float(v0[j * 8 + 0]), __uint_as_float(v0[j * 8 + 1]));
          q.y = pack2<T>(__uint_as_float(v0[j * 8 + 2]), __uint_as_float(v0[j * 8 + 3]));
          q.z = pack2<T>(__uint_as_float(v0[j * 8 + 4]), __uint_as_float(v0[j * 8 + 5]));
          q.w = pack2<T>(__uint_as_float(v0[j * 8 + 6]), __uint_as_float(v0[j * 8 + 7]));
          *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = q;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 q;
          q.x = pack2<T>(__uint_as_float(v1[j * 8 + 0]), __uint_as_float(v1[j * 8 + 1]));
          q.y = pack2<T>(__uint_as_float(v1[j * 8 + 2]), __uint_as_float(v1[j * 8 + 3]));
          q.z = pack2<T>(__uint_as_float(v1[j * 8 + 4]), __uint_as_float(v1[j * 8 + 5]));
          q.w = pack2<T>(__uint_as_float(v1[j * 8 + 6]), __uint_as_float(v1[j * 8 + 7]));
          *reinterpret_cast<uint4*>(row + (((j + 4) ^ (lane & 7)) << 4)) = q;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int x = n0 + c * 64;
          const int y = m0 + ew * 32;
          if (x < N && y < M) {
            tma_store_2d(&tm_c, buf, x, y);
          }
          tma_store_commit();
        }
      }
    }
    if (lane == 0) {
      tma_store_wait_all<0>();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// ------------------------------------------------------------ CTA pairs ----
//
// Same pipeline for a cluster of two CTAs that share one 256x256 output tile
// (tcgen05.mma.cta_group::2): CTA r of the pair loads the 128 rows r*128.. of A
// and the 128 columns r*128.. of B, so every operand byte is fetched from L2
// once per pair instead of once per CTA.  A CTA streams 32 KB per k-step instead
// of 48 KB, which is what the single-CTA kernel is limited by.  Only the even
// CTA issues MMAs; the TMA loads of both CTAs signal its `full` barrier, and its
// commits arrive on the `empty` / `tmem_full` barriers of both CTAs.
#ifdef LLMMM_PROFILE
// Debug build only: cycle counters of the MMA thread of CTA 0 (total, waiting for operands,
// waiting for a free accumulator, K-steps), read back with llmmm_profile_dump().
__device__ long long g_prof16[8];
#endif

namespace fp16pair {
constexpr int      BM          = 256;  // per pair; 128 per CTA
constexpr int      BN          = 256;
constexpr int      BK          = 64;
constexpr int      UMMA_K      = 16;
constexpr int      STAGES      = 6;
constexpr int      THREADS     = 256;
constexpr uint32_t A_BYTES     = 128 * BK * 2;             // 16 KB: this CTA's rows
constexpr uint32_t B_BOX_BYTES = 64 * BK * 2;              // 8 KB
constexpr uint32_t B_BYTES     = B_BOX_BYTES * 2;          // 16 KB: this CTA's 128 columns
constexpr uint32_t STAGE_TX    = 2 * (A_BYTES + B_BYTES);  // both CTAs' loads land on the leader's barrier
constexpr uint32_t C_WARP_BUF  = 32 * 128;
constexpr uint32_t OFF_A       = 0;
constexpr uint32_t OFF_B       = OFF_A + STAGES * A_BYTES;
constexpr uint32_t OFF_C       = OFF_B + STAGES * B_BYTES;
constexpr uint32_t OFF_BAR     = OFF_C + 4 * 2 * C_WARP_BUF;
constexpr uint32_t SMEM_BYTES  = OFF_BAR + 256 + 1024;
constexpr uint32_t TMEM_COLS   = 512;
}  // namespace fp16pair

struct Fp16PairBars {
  uint64_t full[fp16pair::STAGES];
  uint64_t empty[fp16pair::STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t fix[4];  // one per epilogue warp: the other chunk of a split tile has landed in shared memory
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// SPLIT = false: every tile is whole; the code for the chunks of a cut tile (and its registers: that epilogue is what
// drove the kernel to 255 registers and a spill) is left out.  The launcher picks the instantiation from its plan.
template<typename T, bool SPLIT>
__global__ void __launch_bounds__(fp16pair::THREADS, 1)
  fp16_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                        const __grid_constant__ CUtensorMap tm_b,
                        const __grid_constant__ CUtensorMap tm_c,
                        int                                 M,
                        int                                 N,
                        int                                 K,
                        int                                 dp_tiles,
                        int                                 split_pairs,
                        int                                 split_s,
                        int                                 split_chunk,
                        float* __restrict__                 sk_partials,
                        uint32_t* __restrict__              sk_counters,
                        uint32_t*                           status)
{
  using namespace fp16pair;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Fp16PairBars*      bars       = reinterpret_cast<Fp16PairBars*>(smem + OFF_BAR);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int      warp     = threadIdx.x >> 5;
  const int      lane     = threadIdx.x & 31;
  const uint32_t rank     = cluster_ctarank();  // 0 = leader
  const int      pair     = blockIdx.x >> 1;
  const int      n_pairs  = gridDim.x >> 1;

  const int m_tiles = (M + BM - 1) / BM;
  const int k_iters = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 8);  // 4 epilogue warps of each CTA
    }
    for (int w = 0; w < 4; ++w) {
      mbar_init(&bars->fix[w], 1);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b);
    prefetch_tmap(&tm_c);
  }
  if (warp == 2) {
    tmem_alloc<TMEM_COLS>(&bars->tmem_base);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the pair's barriers exist before any cross-CTA signal
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // no global memory touched so far: this may overlap the tail of the previous kernel on the stream
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      uint32_t it = 0;
      PairWalk walk(pair, n_pairs, k_iters, dp_tiles, split_pairs, split_s, split_chunk);
      int      tile, kb0, kb1;
      while (walk.next(tile, kb0, kb1)) {
        const int m0 = (tile % m_tiles) * BM + (int)rank * 128;
        const int n0 = (tile / m_tiles) * BN + (int)rank * 128;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s  = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          mbar_wait(&bars->empty[s], ph ^ 1, DEV_WAIT_SMEM_EMPTY, abort_flag, status);
          const uint32_t full_leader = mapa_shared(smem_u32(&bars->full[s]), 0);
          if (rank == 0) {
            mbar_arrive_expect_tx(&bars->full[s], STAGE_TX);
          }
          tma_load_2d_pair(smem + OFF_A + s * A_BYTES, &tm_a, full_leader, kb * BK, m0);
          tma_load_2d_pair(smem + OFF_B + s * B_BYTES, &tm_b, full_leader, n0, kb * BK);
          tma_load_2d_pair(smem + OFF_B + s * B_BYTES + B_BOX_BYTES, &tm_b, full_leader, n0 + 64, kb * BK);
        }
      }
    }
  }
  else if (warp == 1) {
    // ------------------------------------------- MMA issuer (leader only) --
    if (lane == 0 && rank == 0) {
      constexpr uint32_t kFmt  = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = make_idesc(kFmt, kFmt, /*a_mn=*/0, /*b_mn=*/1, BM, BN);
      uint32_t           it    = 0;
      uint32_t           t     = 0;
#ifdef LLMMM_PROFILE
      long long p_t0 = clock64(), p_full = 0, p_tmem = 0;
      unsigned long long p_g0 = global_timer_ns();
#define PROF_T(x) long long x = clock64()
#else
#define PROF_T(x)
#endif
      PairWalk walk(pair, n_pairs, k_iters, dp_tiles, split_pairs, split_s, split_chunk);
      int      tile, kb0, kb1;
      for (; walk.next(tile, kb0, kb1); ++t) {
        const uint32_t acc    = t & 1;
        const uint32_t acc_ph = (t >> 1) & 1;
        PROF_T(c0);
        mbar_wait(&bars->tmem_empty[acc], acc_ph ^ 1, DEV_WAIT_TMEM_EMPTY, abort_flag, status);
        PROF_T(c1);
#ifdef LLMMM_PROFILE
        p_tmem += c1 - c0;
#endif
        tc_fence_after_sync();
        const uint32_t d_addr = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s  = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          PROF_T(c2);
          mbar_wait(&bars->full[s], ph, DEV_WAIT_SMEM_FULL, abort_flag, status);
          PROF_T(c3);
#ifdef LLMMM_PROFILE
          p_full += c3 - c2;
#endif
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(smem_u32(smem + OFF_A + s * A_BYTES), 0, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_u32(smem + OFF_B + s * B_BYTES), B_BOX_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            tc_mma_f16_pair(d_addr,
                            da + (uint64_t)((kk * UMMA_K * 2) >> 4),
                            db + (uint64_t)((kk * UMMA_K * 128) >> 4),
                            idesc,
                            (kb != kb0) || (kk != 0));
          }
          tc_commit_pair(&bars->empty[s]);
        }
        tc_commit_pair(&bars->tmem_full[acc]);
      }
#ifdef LLMMM_PROFILE
      if (blockIdx.x == 0) {
        g_prof16[0] = clock64() - p_t0;
        g_prof16[1] = (long long)(global_timer_ns() - p_g0);
        g_prof16[2] = p_full;
        g_prof16[3] = p_tmem;
        g_prof16[4] = it;
      }
#endif
    }
  }
  else if (warp >= 4) {
    // ---------------------------------------------------------- epilogue --
    const int      ew           = warp - 4;
    uint8_t*       cbuf         = smem + OFF_C + ew * 2 * C_WARP_BUF;
    uint32_t       t            = 0;
    uint32_t       chunk_it     = 0;
    // 64 fp32 values per lane (row `lane`, columns n0 + c*64 ..) -> T, through this warp's swizzled
    // staging buffer, out with one TMA store
    auto convert_and_store = [&](const uint32_t(&v0)[32], const uint32_t(&v1)[32], int m0, int n0, int c) {
      uint8_t* buf = cbuf + (chunk_it & 1) * C_WARP_BUF;
      if (lane == 0) {
        tma_store_wait_read<1>();
      }
      __syncwarp();
      uint8_t* row = buf + lane * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 q;
        q.x = pack2<T>(__uint_as_float(v0[j * 8 + 0]), __uint_as_float(v0[j * 8 + 1]));
        q.y = pack2<T>(__uint_as_float(v0[j * 8 + 2]), __uint_as_float(v0[j * 8 + 3]));
        q.z = pack2<T>(__uint_as_float(v0[j * 8 + 4]), __uint_as_float(v0[j * 8 + 5]));
        q.w = pack2<T>(__uint_as_float(v0[j * 8 + 6]), __uint_as_float(v0[j * 8 + 7]));
        *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = q;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 q;
        q.x = pack2<T>(__uint_as_float(v1[j * 8 + 0]), __uint_as_float(v1[j * 8 + 1]));
        q.y = pack2<T>(__uint_as_float(v1[j * 8 + 2]), __uint_as_float(v1[j * 8 + 3]));
        q.z = pack2<T>(__uint_as_float(v1[j * 8 + 4]), __uint_as_float(v1[j * 8 + 5]));
        q.w = pack2<T>(__uint_as_float(v1[j * 8 + 6]), __uint_as_float(v1[j * 8 + 7]));
        *reinterpret_cast<uint4*>(row + (((j + 4) ^ (lane & 7)) << 4)) = q;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int x = n0 + c * 64;
        const int y = m0 + ew * 32;
        if (x < N && y < M) {
          tma_store_2d(&tm_c, buf, x, y);
        }
        tma_store_commit();
      }
      ++chunk_it;
    };
    auto release_accumulator = [&](uint32_t acc) {
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(mapa_shared(smem_u32(&bars->tmem_empty[acc]), 0));
      }
    };

    PairWalk walk(pair, n_pairs, k_iters, dp_tiles, split_pairs, split_s, split_chunk);
    int      tile, kb0, kb1;
    for (; walk.next(tile, kb0, kb1); ++t) {
      const int      m0     = (tile % m_tiles) * BM + (int)rank * 128;
      const int      n0     = (tile / m_tiles) * BN;
      const uint32_t acc    = t & 1;
      const uint32_t acc_ph = (t >> 1) & 1;
      mbar_wait(&bars->tmem_full[acc], acc_ph, DEV_WAIT_TMEM_FULL, abort_flag, status);
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(ew * 32) << 16);
      if (!SPLIT || kb1 - kb0 == k_iters) {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(t_addr + c * 64, v0);
          tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
          tmem_ld_wait();
          if (c == BN / 64 - 1) {
            // the accumulator is drained: tell the leader's MMA thread
            release_accumulator(acc);
          }
          convert_and_store(v0, v1, m0, n0, c);
        }
        continue;
      }
      if constexpr (SPLIT) {
      // A chunk of a split tile, the last piece of work of this pair.  This warp's 32x256 piece is handled
      // independently of the other warps: publish the fp32 partial sums (four columns per lane side by
      // side: 512 contiguous bytes per warp instruction), count the arrival, and if it is the last one
      // for this piece, add all chunks in the order of their K ranges (this pair's own chunk is still in
      // tensor memory) and write the tile.  Nothing here waits for another CTA.
      const int      tt   = tile - dp_tiles;
      const uint32_t unit = rank * 4 + (uint32_t)ew;
      constexpr size_t   UNIT_FLOAT4 = SPLIT_SLOT_FLOATS / 8 / 4;  // 8 units of 32 rows x 256 columns per slot
      constexpr uint32_t UNIT_BYTES  = (uint32_t)(UNIT_FLOAT4 * 16);
      static_assert(4 * UNIT_BYTES <= OFF_C, "the four staging units must fit into the operand ring");
      // The operand ring is idle (the last MMAs of this CTA pair are done): this warp's 32 KB of it stage
      // the piece on its way out and, for the warp that sums, the other chunk on its way in.  Bulk copies
      // move a piece about three times faster than the load/store units do (measured: 128 KB per CTA in
      // 2.2 us with 16-byte stores).
      float4* stage = reinterpret_cast<float4*>(smem + OFF_A + (uint32_t)ew * UNIT_BYTES) + lane;
      float*  mine  = sk_partials + (size_t)pair * SPLIT_SLOT_FLOATS + unit * (UNIT_FLOAT4 * 4);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_addr + c * 64, v0);
        tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          stage[(c * 16 + j) * 32] = make_float4(__uint_as_float(v0[4 * j]), __uint_as_float(v0[4 * j + 1]),
                                                 __uint_as_float(v0[4 * j + 2]), __uint_as_float(v0[4 * j + 3]));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          stage[(c * 16 + 8 + j) * 32] = make_float4(__uint_as_float(v1[4 * j]), __uint_as_float(v1[4 * j + 1]),
                                                     __uint_as_float(v1[4 * j + 2]), __uint_as_float(v1[4 * j + 3]));
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      uint32_t arrived = 0;
      if (lane == 0) {
        bulk_store(mine, stage, UNIT_BYTES);
        tma_store_commit();
        tma_store_wait_all<0>();  // written, not merely read out of shared memory
        fence_proxy_async_all();
        __threadfence();
        arrived = atomicAdd(&sk_counters[tt * 16 + unit], 1u);
      }
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (arrived == (uint32_t)(split_s - 1)) {
        __threadfence();
        const int my_chunk = pair % split_s;
        if (split_s == 2) {
          // two chunks: a + b == b + a bit for bit; this pair's chunk is still in tensor memory, the other
          // one comes in with one bulk copy
          if (lane == 0) {
            fence_proxy_async_all();
            mbar_arrive_expect_tx(&bars->fix[ew], UNIT_BYTES);
            bulk_load(stage, sk_partials + (size_t)(pair ^ 1) * SPLIT_SLOT_FLOATS + unit * (UNIT_FLOAT4 * 4), UNIT_BYTES,
                      &bars->fix[ew]);
          }
          mbar_wait(&bars->fix[ew], 0, DEV_WAIT_TMEM_FULL, abort_flag, status);
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t s0[32], s1[32];
            tmem_ld_32x32b_x32(t_addr + c * 64, s0);
            tmem_ld_32x32b_x32(t_addr + c * 64 + 32, s1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 a = stage[(c * 16 + j) * 32];
              const float4 b = stage[(c * 16 + 8 + j) * 32];
              s0[4 * j]     = __float_as_uint(__uint_as_float(s0[4 * j]) + a.x);
              s0[4 * j + 1] = __float_as_uint(__uint_as_float(s0[4 * j + 1]) + a.y);
              s0[4 * j + 2] = __float_as_uint(__uint_as_float(s0[4 * j + 2]) + a.z);
              s0[4 * j + 3] = __float_as_uint(__uint_as_float(s0[4 * j + 3]) + a.w);
              s1[4 * j]     = __float_as_uint(__uint_as_float(s1[4 * j]) + b.x);
              s1[4 * j + 1] = __float_as_uint(__uint_as_float(s1[4 * j + 1]) + b.y);
              s1[4 * j + 2] = __float_as_uint(__uint_as_float(s1[4 * j + 2]) + b.z);
              s1[4 * j + 3] = __float_as_uint(__uint_as_float(s1[4 * j + 3]) + b.w);
            }
            convert_and_store(s0, s1, m0, n0, c);
          }
        }
        else {
          // more chunks: added in the order of their K ranges, read with plain loads
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t s0[32], s1[32];
#pragma unroll 1
            for (int w = 0; w < split_s; ++w) {
              uint32_t v0[32], v1[32];
              if (w == my_chunk) {
                tmem_ld_32x32b_x32(t_addr + c * 64, v0);
                tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
                tmem_ld_wait();
              }
              else {
                const float4* src = reinterpret_cast<const float4*>(sk_partials + (size_t)(tt * split_s + w) * SPLIT_SLOT_FLOATS)
                                    + unit * UNIT_FLOAT4 + lane;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 a = __ldcg(src + (c * 16 + j) * 32);
                  const float4 b = __ldcg(src + (c * 16 + 8 + j) * 32);
                  v0[4 * j]     = __float_as_uint(a.x);
                  v0[4 * j + 1] = __float_as_uint(a.y);
                  v0[4 * j + 2] = __float_as_uint(a.z);
                  v0[4 * j + 3] = __float_as_uint(a.w);
                  v1[4 * j]     = __float_as_uint(b.x);
                  v1[4 * j + 1] = __float_as_uint(b.y);
                  v1[4 * j + 2] = __float_as_uint(b.z);
                  v1[4 * j + 3] = __float_as_uint(b.w);
                }
              }
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                s0[i] = (w == 0) ? v0[i] : __float_as_uint(__uint_as_float(s0[i]) + __uint_as_float(v0[i]));
                s1[i] = (w == 0) ? v1[i] : __float_as_uint(__uint_as_float(s1[i]) + __uint_as_float(v1[i]));
              }
            }
            convert_and_store(s0, s1, m0, n0, c);
          }
        }
        if (lane == 0) {
          sk_counters[tt * 16 + unit] = 0;  // every launch leaves the counters at zero
        }
      }
      release_accumulator(acc);
      }  // SPLIT
    }
    if (lane == 0) {
      tma_store_wait_all<0>();
    }
  }

  // neither CTA may leave while its partner can still signal its barriers or read its tiles
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

template<typename T>
static int launch_fp16_pair(const void* A, const void* B, void* C, int M, int N, int K, const DeviceInfo* info, cudaStream_t stream)
{
  using namespace fp16pair;
  constexpr CUtensorMapDataType dt =
    std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_a, tm_b, tm_c;
  if (!make_tmap_2d(&tm_a, A, dt, 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_b, B, dt, 2, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_c, C, dt, 2, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(
      cudaFuncSetAttribute(fp16_gemm_pair_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    LLMMM_CUDA_TRY(
      cudaFuncSetAttribute(fp16_gemm_pair_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    attr_set[info->device] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  // estimated cost of a split, in K-steps of 64 (one takes about 0.33 us): publishing a chunk and counting
  // the arrival about 3 us, reading a chunk back about 1.5 us
  const SplitPlan plan = plan_split(info, tiles, (K + BK - 1) / BK, /*fixed*/ 10, /*per_way_x2*/ 9, /*min_gain*/ 6);
  if (plan.split_pairs > 0) {
    LLMMM_CUDA_TRY(launch_pdl(fp16_gemm_pair_kernel<T, true>, dim3(2 * plan.pairs), dim3(THREADS), SMEM_BYTES, stream, 2, tm_a,
                              tm_b, tm_c, M, N, K, plan.dp_tiles, plan.split_pairs, plan.split_s, plan.split_chunk,
                              plan.partials, plan.counters, info->status));
  }
  else {
    LLMMM_CUDA_TRY(launch_pdl(fp16_gemm_pair_kernel<T, false>, dim3(2 * plan.pairs), dim3(THREADS), SMEM_BYTES, stream, 2, tm_a,
                              tm_b, tm_c, M, N, K, plan.dp_tiles, plan.split_pairs, plan.split_s, plan.split_chunk,
                              plan.partials, plan.counters, info->status));
  }
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

// Which kernel a problem runs on: more than 128 rows (and columns) the pair kernel; 65..128 rows the single-CTA
// kernel, unless its tiles would occupy at most half of the SMs and scratch is registered: then the pair
// kernel, whose tiles can be cut along K (the same rule as for FP8).
static bool fp16_use_pair_kernel(const DeviceInfo* info, int M, int N)
{
  if (info->max_pairs < 1 || N <= 128) {
    return false;
  }
  if (M > 128) {
    return true;
  }
  const int       tiles_1cta = ((M + fp16cfg::BM - 1) / fp16cfg::BM) * ((N + fp16cfg::BN - 1) / fp16cfg::BN);
  const Workspace ws         = registered_workspace(info->device);
  return M > 64 && ws.ptr != nullptr && ws.bytes >= split_workspace_bytes() && 2 * tiles_1cta <= info->sm_count;
}

void describe_fp16_plan(const DeviceInfo* info, bool bf16, int M, int N, int K, char* buf, size_t len)
{
  const char* t = bf16 ? "__nv_bfloat16" : "__half";
  if (fp16_use_pair_kernel(info, M, N)) {
    using namespace fp16pair;
    const int       tiles   = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int       k_steps = (K + BK - 1) / BK;
    const SplitPlan plan    = plan_split(info, tiles, k_steps, 10, 9, 6, false);
    if (plan.split_pairs > 0) {
      snprintf(buf, len, "fp16_gemm_pair_kernel<%s>: %d tiles of 256x256 on %d CTA pairs; %d whole tiles round-robin, then %d "
               "tiles cut %d-way along K (chunks of %d k-steps of 64), one chunk per pair", t, tiles, plan.pairs, plan.dp_tiles,
               tiles - plan.dp_tiles, plan.split_s, plan.split_chunk);
    }
    else {
      snprintf(buf, len, "fp16_gemm_pair_kernel<%s>: %d tiles of 256x256 on %d CTA pairs (%.2f waves), %d k-steps of 64 each, "
               "no split", t, tiles, plan.pairs, (double)tiles / plan.pairs, k_steps);
    }
    return;
  }
  using namespace fp16cfg;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid  = tiles < info->sm_count ? tiles : info->sm_count;
  snprintf(buf, len, "fp16_gemm_kernel<%s>: %d tiles of %dx%d on %d CTAs (%.2f waves)", t, tiles, BM, BN, grid, (double)tiles / grid);
}

int warm_fp16_kernels(const DeviceInfo* info)
{
  (void)info;
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp16_gemm_pair_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp16pair::SMEM_BYTES));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp16_gemm_pair_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp16pair::SMEM_BYTES));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp16_gemm_pair_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp16pair::SMEM_BYTES));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp16_gemm_pair_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp16pair::SMEM_BYTES));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp16_gemm_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp16cfg::SMEM_BYTES));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp16_gemm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp16cfg::SMEM_BYTES));
  return LLMMM_OK;
}

template<typename T>
static int launch_fp16(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t stream)
{
  using namespace fp16cfg;
  if (A == nullptr || B == nullptr || C == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (M < 1 || N < 8 || K < 8 || (N % 8) != 0 || (K % 8) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "M or N or K are not aligned. (need M>=1, N%%8==0, K%%8==0; got %d %d %d)", M, N, K);
  }
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "A, B and C must be 16-byte aligned");
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  constexpr CUtensorMapDataType dt =
    std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_a, tm_b, tm_c;
  if (!make_tmap_2d(&tm_a, A, dt, 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_b, B, dt, 2, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_c, C, dt, 2, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  if (fp16_use_pair_kernel(info, M, N)) {
    return launch_fp16_pair<T>(A, B, C, M, N, K, info, stream);
  }
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(
      cudaFuncSetAttribute(fp16_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    attr_set[info->device] = true;
  }
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = (N + BN - 1) / BN;
  const int tiles   = m_tiles * n_tiles;
  const int grid    = tiles < info->sm_count ? tiles : info->sm_count;
  LLMMM_CUDA_TRY(launch_pdl(fp16_gemm_kernel<T>, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, 1, tm_a, tm_b, tm_c, M, N, K,
                            info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

}  // namespace llmmm

#ifdef LLMMM_PROFILE
extern "C" void llmmm_profile_dump16()
{
  long long h[8];
  cudaMemcpyFromSymbol(h, llmmm::g_prof16, sizeof(h));
  printf("fp16 pair kernel, CTA 0 MMA thread: %.3f GHz, %.1f us, %lld k-steps, %.0f clk/k-step, waiting operands %.0f, waiting accumulator %.0f clk/k-step\n",
         (double)h[0] / h[1], h[1] / 1e3, h[4], (double)h[0] / h[4], (double)h[2] / h[4], (double)h[3] / h[4]);
}
#endif

extern "C" {

int llmmm_fp16_mm_f16(const void* A, const void* B, void* C, int M, int N, int K, llmmm_stream_t stream)
{
  return llmmm::launch_fp16<__half>(A, B, C, M, N, K, reinterpret_cast<cudaStream_t>(stream));
}

int llmmm_fp16_mm_bf16(const void* A, const void* B, void* C, int M, int N, int K, llmmm_stream_t stream)
{
  return llmmm::launch_fp16<__nv_bfloat16>(A, B, C, M, N, K, reinterpret_cast<cudaStream_t>(stream));
}

int llmmm_fp16_mm_f16_ws(const void* A, const void* B, void* C, int M, int N, int K, void* workspace, size_t workspace_bytes,
                         llmmm_stream_t stream)
{
  const int rc = llmmm::check_workspace_arg(workspace, workspace_bytes);
  if (rc != LLMMM_OK) {
    return rc;
  }
  llmmm::ScopedWorkspace bound(workspace, workspace_bytes);
  return llmmm::launch_fp16<__half>(A, B, C, M, N, K, reinterpret_cast<cudaStream_t>(stream));
}

int llmmm_fp16_mm_bf16_ws(const void* A, const void* B, void* C, int M, int N, int K, void* workspace, size_t workspace_bytes,
                          llmmm_stream_t stream)
{
  const int rc = llmmm::check_workspace_arg(workspace, workspace_bytes);
  if (rc != LLMMM_OK) {
    return rc;
  }
  llmmm::ScopedWorkspace bound(workspace, workspace_bytes);
  return llmmm::launch_fp16<__nv_bfloat16>(A, B, C, M, N, K, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
