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
//     e4m3 and write their 128 bytes into the warp's 4 KB staging tile in
//     shared memory (128-byte swizzle), which one lane hands to a TMA store:
//     the tile leaves as whole rows (a thread storing its own row would make
//     every store instruction of the warp touch 32 rows); the scale column is
//     stored directly, it is coalesced.
#include <cuda_fp8.h>

#include "host_common.h"
#include "pair_walk.cuh"
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
// setmaxnreg moves registers inside the CTA's allocation (the 168 per thread ptxas reports for 384 threads); a
// split that asks for more than that makes setmaxnreg.inc wait for ever
static_assert(128 * REGS_CTRL + 256 * REGS_PROMO <= THREADS * 168, "setmaxnreg split exceeds the CTA's registers");
constexpr uint32_t A_BYTES    = BM * BK;
constexpr uint32_t B_BYTES    = BN * BK;
constexpr uint32_t STAGE_TX   = A_BYTES + B_BYTES;
constexpr uint32_t OFF_A      = 0;
constexpr uint32_t OFF_B      = OFF_A + STAGES * A_BYTES;
constexpr uint32_t OFF_BAR    = OFF_B + STAGES * B_BYTES;
constexpr uint32_t OFF_STG    = OFF_BAR + 1024;  // eight 4 KB staging tiles: a promotion warp's 32 rows x 128 output bytes
constexpr uint32_t SMEM_BYTES = OFF_STG + 8 * 4096 + 1024;
static_assert(SMEM_BYTES <= 232448, "ring + staging tiles exceed the shared memory of an SM");
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

// acc{0,1} = fma(v{0,1}, sc, acc{0,1}).  Two scalar FMAs: the packed fma.rn.f32x2 has the same flop rate
// and was measured slower here (aligned register pairs cost registers in a loop that has none to spare).
__device__ __forceinline__ void ffma2(float& d0, float& d1, uint32_t a0, uint32_t a1, float sc)
{
  d0 = __fmaf_rn(__uint_as_float(a0), sc, d0);
  d1 = __fmaf_rn(__uint_as_float(a1), sc, d1);
}

// largest magnitude of a thread's 128 accumulators, in four chains (one chain is 128 dependent instructions)
__device__ __forceinline__ float amax128(const float (&acc)[128])
{
  float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < 128; ++i) {
    a[i & 3] = fmaxf(a[i & 3], fabsf(acc[i]));
  }
  return fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
}

// Shared-memory address of a generic pointer, computed where this stands (asm volatile is not hoisted above the
// barrier waits of a loop in front of it).
__device__ __forceinline__ uint32_t smem_u32_pinned(const void* p)
{
  uint32_t a;
  asm volatile("{\n.reg .u64 t;\ncvta.to.shared.u64 t, %1;\ncvt.u32.u64 %0, t;\n}" : "=r"(a) : "l"(p));
  return a;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w)
{
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// tma_store_2d with the source given as a shared-memory address
__device__ __forceinline__ void tma_store_2d_from(const CUtensorMap* m, uint32_t src, int x, int y)
{
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
               : "memory");
}

// OUT_F32 = false: C_q e4m3 + C_s;  true: C fp32, no quantisation.
template<bool OUT_F32>
__global__ void __launch_bounds__(fp8cfg::THREADS, 1) fp8_blockwise_gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                                                const __grid_constant__ CUtensorMap tm_b,
                                                                                const __grid_constant__ CUtensorMap tm_c,  // e4m3 output: C as [M, N] bytes, boxes of 32 rows x 128
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
    if constexpr (!OUT_F32) {
      prefetch_tmap(&tm_c);
    }
  }
  if (warp == 1) {
    tmem_alloc<TMEM_COLS>(&bars->tmem_base);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // no global memory touched so far: this may overlap the tail of the previous kernel on the stream
  pdl_launch_dependents();
  pdl_wait();

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
      constexpr int PREFETCH = 2;
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
        const float    sc  = __fmul_rn(a_cur, b_cur);
        const float    sc2 = sc;
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
        for (int i = 0; i < 32; i += 2) {
          ffma2(acc[i], acc[i + 1], v0[i], v0[i + 1], sc2);
        }
        tmem_ld_wait();
        tmem_ld_32x32b_x32(t_addr + 64, v0);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          ffma2(acc[32 + i], acc[32 + i + 1], v1[i], v1[i + 1], sc2);
        }
        tmem_ld_wait();
        tmem_ld_32x32b_x32(t_addr + 96, v1);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          ffma2(acc[64 + i], acc[64 + i + 1], v0[i], v0[i + 1], sc2);
        }
        tmem_ld_wait();
        // every column of this thread's part of the partial stage has been read
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->part_empty[p]);
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          ffma2(acc[96 + i], acc[96 + i + 1], v1[i], v1[i + 1], sc2);
        }
        ++it;
      }
      }

      // The warp's 32 output rows go through a 4 KB staging tile (16-byte chunks XOR-swizzled by row = the
      // 128-byte swizzle of the tensor map) and leave as TMA stores of whole rows; written directly, every store
      // instruction would touch 32 rows.  All lanes take part; rows beyond M are clipped by the tensor map.
      // (the tile's shared-memory address is derived here from scratch: the K loop has no register to carry it)
      const uint32_t stg      = ((smem_u32_pinned(smem_raw) + 1023u) & ~1023u) + OFF_STG + (uint32_t)(warp - 4) * 4096u;
      const bool     store_ok = g_ok && m - lane < M;
      (void)stg;
      (void)store_ok;
      if constexpr (OUT_F32) {
        // (fp32 rows are written directly: the staged form of the pair kernel does not fit this kernel's registers)
        if (m_ok && g_ok) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(C_out) + (size_t)m * N + (size_t)ng * 128);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
          }
        }
      }
      else {
        const float amax      = amax128(acc);
        const float scale     = __fdiv_rn(amax, 448.0f);
        const float scale_inv = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
        tma_store_wait_read<0>();  // lane 0: the store of the previous tile has read the staging tile
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 q;
          q.x = pack_e4m3x4(acc[16 * i + 0] * scale_inv, acc[16 * i + 1] * scale_inv, acc[16 * i + 2] * scale_inv, acc[16 * i + 3] * scale_inv);
          q.y = pack_e4m3x4(acc[16 * i + 4] * scale_inv, acc[16 * i + 5] * scale_inv, acc[16 * i + 6] * scale_inv, acc[16 * i + 7] * scale_inv);
          q.z = pack_e4m3x4(acc[16 * i + 8] * scale_inv, acc[16 * i + 9] * scale_inv, acc[16 * i + 10] * scale_inv, acc[16 * i + 11] * scale_inv);
          q.w = pack_e4m3x4(acc[16 * i + 12] * scale_inv, acc[16 * i + 13] * scale_inv, acc[16 * i + 14] * scale_inv, acc[16 * i + 15] * scale_inv);
          sts128(stg + lane * 128 + ((i ^ (lane & 7)) << 4), q.x, q.y, q.z, q.w);
        }
        if (m_ok && g_ok) {
          C_s[(size_t)ng * M + m] = scale;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && store_ok) {
          tma_store_2d_from(&tm_c, stg, ng * 128, m - lane);
          tma_store_commit();
        }
      }
    }
    if (!OUT_F32 && lane == 0) {
      tma_store_wait_read<0>();  // shared memory must outlive the last store's read of it
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// ------------------------------------------------------------ CTA pairs ----
//
// The same computation for a cluster of two CTAs that share one 256x256 output
// tile (tcgen05.mma.cta_group::2), used when M > 128.  CTA r loads its own 128
// rows of A_q and the 128 B_q rows of the tile's scale group r, so a CTA
// streams 32 KB per K-block instead of 48 KB (6-stage ring) and its shared
// memory serves 32 KB of operand reads per K-block instead of 48 KB.  Shared
// memory bandwidth (TMA writes + MMA reads, about 128 B/clk) is what bounds the
// single-CTA kernel.  Only the even CTA issues MMAs (256x256x32); both CTAs'
// loads signal its `full` barrier, its commits arrive on both CTAs' `empty` and
// `part_full` barriers, and both CTAs' promotion warps release a partial stage
// by arriving on its `part_empty` barrier.
#ifdef LLMMM_PROFILE
// Debug build only: cycle counters of CTA 0 (MMA thread: total, waiting for operands, waiting for a
// free partial stage; promotion warp 4: waiting for a partial, epilogue), see llmmm_profile_dump8().
__device__ long long g_prof8[16];
__device__ long long g_trace8[64][8];  // per K-block of CTA 0: clock64 at the hand-off points
__device__ unsigned long long g_stamp8[4][16];  // split-tile hand-offs of promotion warp 4 of CTAs 0..3 (ns)
#define PROF8_T(x) long long x = clock64()
#define PROF8_ADD(dst, a, b) dst += (b) - (a)
#define PROF8_STAMP(i)                                                                                                 \
  if (blockIdx.x < 4 && threadIdx.x == 128) {                                                                          \
    g_stamp8[blockIdx.x][i] = global_timer_ns();                                                                       \
  }
#else
#define PROF8_T(x)
#define PROF8_ADD(dst, a, b)
#define PROF8_STAMP(i)
#endif

namespace fp8pair {
constexpr int      BM         = 256;  // per pair; 128 rows per CTA
constexpr int      BN         = 256;
constexpr int      BK         = 128;
constexpr int      UMMA_K     = 32;
constexpr int      STAGES     = 6;
constexpr int      THREADS    = 384;
constexpr int      REGS_CTRL  = 32;  // 32/232 compiles without spills; 40/232 spilt in the promotion loop (+35 % time)
constexpr int      REGS_PROMO = 232;
static_assert(128 * REGS_CTRL + 256 * REGS_PROMO <= THREADS * 168, "setmaxnreg split exceeds the CTA's registers");
constexpr uint32_t A_BYTES    = 128 * BK;                 // 16 KB: this CTA's rows
constexpr uint32_t B_BYTES    = 128 * BK;                 // 16 KB: this CTA's half of the tile's columns
constexpr uint32_t STAGE_TX   = 2 * (A_BYTES + B_BYTES);  // both CTAs' loads land on the leader's barrier
constexpr uint32_t OFF_A      = 0;
constexpr uint32_t OFF_B      = OFF_A + STAGES * A_BYTES;
constexpr uint32_t OFF_BAR    = OFF_B + STAGES * B_BYTES;
constexpr uint32_t OFF_XCH    = OFF_BAR + 256;  // 2 x 256 floats: row maxima exchanged between the column halves (SWIGLU)
// The e4m3 epilogues transpose each promotion warp's 32 x 128-byte output tile through 4 KB of shared memory
// (16-byte chunks XOR-swizzled by row, which is the 128-byte swizzle of a tensor map), so that the tile leaves as
// whole rows: one TMA store per warp (EPI_E4M3) or store instructions that cover four rows each.  EPI_E4M3 and
// EPI_GATHER keep the eight staging tiles from OFF_STG on (1024-byte aligned; SWIGLU's exchange buffer overlaps
// it, that instantiation has no staging tiles).
constexpr uint32_t OFF_STG           = OFF_BAR + 1024;
constexpr uint32_t SMEM_BYTES_STAGED = OFF_STG + 8 * 4096 + 1024;
static_assert(SMEM_BYTES_STAGED <= 232448, "staging tiles + ring exceed the shared memory of an SM");
// EPI_ROPE keeps the angle-table rows of the tile's 128 rows in shared memory: 32 rows x (256 B cos | 256 B sin)
// = 16 KB per row quarter.  Quarters 0 and 1 use the two slots of the ring's sixth stage (the ring runs with
// five), quarters 2 and 3 the 32 KB from OFF_STG on; the two norm weight vectors follow.  Once a tile's rows have
// been used, the first 8 KB of each quarter's region serve as the two staging tiles of its warps.
constexpr uint32_t ROPE_TAB_BYTES  = 32 * 512;
constexpr uint32_t OFF_ROPE_W      = OFF_STG + 2 * ROPE_TAB_BYTES;  // 2 x 128 floats: query and key norm weights
constexpr uint32_t SMEM_BYTES_ROPE = OFF_ROPE_W + 1024 + 1024;

// EPI_SWIGLU: a warp's output tile is 32 rows x 64 bytes (2 KB, 16-byte chunks in the 64-byte swizzle of a tensor
// map); its eight staging tiles lie behind the exchange buffer.
constexpr uint32_t OFF_STG_SWIGLU    = OFF_BAR + 3072;
constexpr uint32_t SMEM_BYTES_SWIGLU = OFF_STG_SWIGLU + 8 * 2048 + 1024;
static_assert(OFF_XCH + 2048 <= OFF_STG_SWIGLU, "exchange buffer and staging tiles overlap");

constexpr uint32_t smem_bytes_of(int epi)  // (the EPI_* constants: 2 swiglu, 4 rope)
{
  return epi == 4 ? SMEM_BYTES_ROPE : epi == 2 ? SMEM_BYTES_SWIGLU : SMEM_BYTES_STAGED;
}
constexpr uint32_t TMEM_COLS  = 512;  // two partial stages of 256 columns
// split tiles (pair_walk.cuh): a slot holds 16 warp-sized units of 32 rows x 128 columns
constexpr size_t   SK_UNIT_FLOATS = 32 * 128;
static_assert(16 * SK_UNIT_FLOATS == SPLIT_SLOT_FLOATS, "one slot per 256x256 tile");
}  // namespace fp8pair

struct Fp8PairBars {
  uint64_t full[fp8pair::STAGES];   // used in the leader CTA
  uint64_t empty[fp8pair::STAGES];  // both CTAs (multicast commit)
  uint64_t part_full[2];            // both CTAs (multicast commit)
  uint64_t part_empty[2];           // used in the leader CTA, 16 arrivals
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// What the pair kernel does with a finished tile:
//   EPI_E4M3   C_q e4m3 + C_s (1x128 groups along N)
//   EPI_F32    C fp32, no quantisation
//   EPI_SWIGLU B_t holds a gate_up weight [2I, K] (gate rows first); a tile covers 128 output columns: CTA r
//              loads gate rows n0 + 64r .. and up rows I + n0 + 64r .., so that a thread's 128 accumulators are
//              64 gate values and the 64 up values of the SAME columns; H = silu(gate) * up is quantised
//              1x128 along I into H_q [M, I] + H_s [I/128, M], the A-operand format of the next GEMM.
//              The kernel's N parameter is I.
//   EPI_GATHER like EPI_E4M3, but this call computes a column shard [col0, col0 + N) of a wider C and stores it
//              into the full C_q [M, ld] / C_s [ld/128, M] of up to 8 destinations at once -- the buffers of the
//              other GPUs of an N-split, mapped into this process: the all-gather of the outputs happens as
//              plain peer stores of the epilogue, overlapped with the tiles still being computed.
//   EPI_ROPE   like EPI_E4M3 for a qkv projection with heads of 128 columns: a thread's 128 accumulators are one
//              head of its row, so the per-head RMSNorm of query / key heads and the rotary embedding are
//              thread-local arithmetic in front of the quantisation.
// Which general kernel a problem runs on.  More than 128 rows: the pair kernel.  65..128 rows: the single-CTA
// kernel (128-row tiles waste nothing), unless its tiles would occupy at most half of the SMs and scratch is
// registered: then the pair kernel, whose tiles can be cut along K, wins although half of each tile's rows are
// empty (measured at M = 128: 2560x9728 45.6 -> 23.6 us, 4096x4096 21.5 -> 18.2 us; 19456x2560, 76 tiles,
// would lose: 17.3 -> 29.3 us).
// With K given, a choice llmmm_tune measured for this weight shape takes precedence (as long as the scratch the
// pair kernel's split needs is there).
static bool fp8_use_pair_kernel(const DeviceInfo* info, int M, int N, int K = 0, bool* tuned = nullptr)
{
  if (tuned != nullptr) {
    *tuned = false;
  }
  if (info->max_pairs < 1) {
    return false;
  }
  if (M > 128) {
    return true;
  }
  if (M <= 64) {
    return false;
  }
  const Workspace ws      = registered_workspace(info->device);
  const bool      scratch = ws.ptr != nullptr && ws.bytes >= split_workspace_bytes();
  if (t_force_mid >= 0) {
    return t_force_mid == 1;
  }
  const int measured = K > 0 ? mid_choice(info->device, N, K) : -1;
  if (measured >= 0 && (measured == 0 || scratch)) {
    if (tuned != nullptr) {
      *tuned = true;
    }
    return measured == 1;
  }
  const int tiles_1cta = ((M + fp8cfg::BM - 1) / fp8cfg::BM) * ((N + fp8cfg::BN - 1) / fp8cfg::BN);
  return scratch && 2 * tiles_1cta <= info->sm_count;
}
constexpr int EPI_E4M3   = 0;
constexpr int EPI_F32    = 1;
constexpr int EPI_SWIGLU = 2;
constexpr int EPI_GATHER = 3;
constexpr int EPI_ROPE   = 4;

struct GatherDst {
  uint8_t* c[8];   // C_q base of every destination
  float*   cs[8];  // C_s base of every destination
  int      n;      // destinations in use
  int      ld;     // columns of the full C
  int      col0;   // first column of this call's shard in the full C
  int      pad;
};

// A read-only 16-byte load the compiler may not move across other asm volatile statements (the epilogue of
// EPI_ROPE limits its loads in flight with it: hoisted above one another they would need a second register file).
__device__ __forceinline__ float4 ldg_pinned(const float4* p)
{
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// the same for shared memory
__device__ __forceinline__ float4 lds_pinned(uint32_t addr)
{
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// 16 bytes from global to shared memory without passing through registers (both addresses 16-byte aligned)
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src)
{
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async_wait_all()
{
  asm volatile("cp.async.wait_all;" ::: "memory");
}

template<int EPI>
__global__ void __launch_bounds__(fp8pair::THREADS, 1)
  fp8_blockwise_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                                 const __grid_constant__ CUtensorMap tm_b,
                                 const __grid_constant__ CUtensorMap tm_c,  // C as rows of bytes, boxes of 32 rows x 128 bytes (SWIGLU: 64; GATHER: unused)
                                 const float* __restrict__ A_s,
                                 const float* __restrict__ B_s,
                                 void* __restrict__ C_out,
                                 float* __restrict__ C_s,
                                 int       M,
                                 int       N,
                                 int       K,
                                 int       dp_tiles,
                                 int       split_pairs,
                                 int       split_s,
                                 int       split_chunk,
                                 float* __restrict__ sk_partials,
                                 uint32_t* __restrict__ sk_counters,
                                 const __grid_constant__ GatherDst gather,
                                 const __grid_constant__ RopeHook rope,
                                 uint32_t* status)
{
  using namespace fp8pair;
  constexpr bool OUT_F32 = (EPI == EPI_F32);
  constexpr bool SWIGLU  = (EPI == EPI_SWIGLU);
  constexpr int  TILE_N  = SWIGLU ? 128 : BN;  // output columns per tile
  // EPI_ROPE runs the ring one stage shorter: the sixth stage's two 16 KB slots hold angle-table rows
  constexpr uint32_t NSTAGES = EPI == EPI_ROPE ? STAGES - 1 : STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Fp8PairBars*       bars       = reinterpret_cast<Fp8PairBars*>(smem + OFF_BAR);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int      warp    = threadIdx.x >> 5;
  const int      lane    = threadIdx.x & 31;
  const uint32_t rank    = cluster_ctarank();
  const int      pair    = blockIdx.x >> 1;
  const int      n_pairs = gridDim.x >> 1;

  const int m_tiles  = (M + BM - 1) / BM;
  const int k_blocks = K / BK;
  const int n_groups = N / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int p = 0; p < 2; ++p) {
      mbar_init(&bars->part_full[p], 1);
      mbar_init(&bars->part_empty[p], 16);  // 8 promotion warps of each CTA
    }
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b);
    if constexpr (EPI != EPI_GATHER) {
      prefetch_tmap(&tm_c);
    }
  }
  if (warp == 2) {
    tmem_alloc<TMEM_COLS>(&bars->tmem_base);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // no global memory touched so far: this may overlap the tail of the previous kernel on the stream
  pdl_launch_dependents();
  pdl_wait();

  if (warp < 4) {
    setmaxnreg_dec<REGS_CTRL>();
    if (warp == 0) {
      // ---------------------------------------------------- TMA producer --
      if (lane == 0) {
        uint32_t it = 0;
        PairWalk walk(pair, n_pairs, k_blocks, dp_tiles, split_pairs, split_s, split_chunk);
        int      tile, kb0, kb1;
        while (walk.next(tile, kb0, kb1)) {
          const int m0 = (tile % m_tiles) * BM + (int)rank * 128;
          const int n0 = (tile / m_tiles) * TILE_N + (int)rank * (SWIGLU ? 64 : 128);
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const uint32_t s  = it % NSTAGES;
            const uint32_t ph = (it / NSTAGES) & 1;
            mbar_wait(&bars->empty[s], ph ^ 1, DEV_WAIT_SMEM_EMPTY, abort_flag, status);
            const uint32_t full_leader = mapa_shared(smem_u32(&bars->full[s]), 0);
            if (rank == 0) {
              mbar_arrive_expect_tx(&bars->full[s], STAGE_TX);
            }
            tma_load_2d_pair(smem + OFF_A + s * A_BYTES, &tm_a, full_leader, kb * BK, m0);
            if constexpr (SWIGLU) {
              // 64 gate rows, then the 64 up rows of the same output columns (the B descriptor's box is 64 rows)
              tma_load_2d_pair(smem + OFF_B + s * B_BYTES, &tm_b, full_leader, kb * BK, n0);
              tma_load_2d_pair(smem + OFF_B + s * B_BYTES + B_BYTES / 2, &tm_b, full_leader, kb * BK, N + n0);
            }
            else {
              tma_load_2d_pair(smem + OFF_B + s * B_BYTES, &tm_b, full_leader, kb * BK, n0);
            }
          }
        }
      }
    }
    else if (warp == 1 || warp == 3) {
      // ------------------------------------ two MMA issuers (leader only) --
      // A thread that issues a group of MMAs followed by tcgen05.commit is held for about the
      // duration of the group (measured: one thread feeds the pipe at 160-190 clk per MMA, two
      // threads issuing alternate groups reach the full 129 clk), and it cannot poll the barriers of
      // the next K-block meanwhile.  Two threads take alternate K-blocks (each owns one TMEM partial
      // stage): one sits in its barrier waits while the MMAs of the other run.
      if (lane == 0 && rank == 0) {
        constexpr uint32_t idesc = make_idesc(/*e4m3*/ 0, 0, 0, 0, BM, BN);
        const uint32_t     p     = (warp == 1) ? 0u : 1u;  // partial stage and K-block parity of this thread
#ifdef LLMMM_PROFILE
        long long p_full = 0, p_part = 0, p_t0 = clock64();
        unsigned long long p_g0 = global_timer_ns();
#endif
        // the MMA threads need no tile identities, only the number of K-blocks this pair works through
        const uint32_t total = PairWalk(pair, n_pairs, k_blocks, dp_tiles, split_pairs, split_s, split_chunk).total_k_blocks();
        for (uint32_t it = p; it < total; it += 2) {
          {
            const uint32_t s  = it % NSTAGES;
            const uint32_t ph = (it / NSTAGES) & 1;
            const uint32_t pp = (it >> 1) & 1;
            PROF8_T(c0);
            mbar_wait(&bars->part_empty[p], pp ^ 1, DEV_WAIT_TMEM_EMPTY, abort_flag, status);
            PROF8_T(c1);
            mbar_wait(&bars->full[s], ph, DEV_WAIT_SMEM_FULL, abort_flag, status);
            PROF8_T(c2);
            PROF8_ADD(p_part, c0, c1);
            PROF8_ADD(p_full, c1, c2);
#ifdef LLMMM_PROFILE
            if (blockIdx.x == 0 && it < 64) {
              g_trace8[it][0] = c0;  // MMA thread: starts waiting for the partial stage
              g_trace8[it][1] = c1;  // partial stage free
              g_trace8[it][2] = c2;  // operands present
            }
#endif
            tc_fence_after_sync();
            const uint64_t da = make_smem_desc_sw128(smem_u32(smem + OFF_A + s * A_BYTES), 0, 1024);
            const uint64_t db = make_smem_desc_sw128(smem_u32(smem + OFF_B + s * B_BYTES), 0, 1024);
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              tc_mma_f8_pair(tmem_base + p * BN, da + (uint64_t)((kk * UMMA_K) >> 4), db + (uint64_t)((kk * UMMA_K) >> 4), idesc, kk != 0);
            }
            tc_commit_pair(&bars->empty[s]);
            tc_commit_pair(&bars->part_full[p]);
#ifdef LLMMM_PROFILE
            if (blockIdx.x == 0 && it < 64) {
              g_trace8[it][3] = clock64();  // MMAs and commits issued
            }
#endif
          }
        }
#ifdef LLMMM_PROFILE
        if (blockIdx.x == 0 && p == 0) {
          g_prof8[0] = clock64() - p_t0;
          g_prof8[1] = (long long)(global_timer_ns() - p_g0);
          g_prof8[2] = 2 * p_full;
          g_prof8[3] = 2 * p_part;
          g_prof8[4] = total;
        }
#endif
      }
    }
  }
  else {
    setmaxnreg_inc<REGS_PROMO>();
    // ------------------------------------------- promotion + epilogue ----
#ifdef LLMMM_PROFILE
    long long p_wait = 0, p_epi = 0, p_p0 = clock64();
#endif
    const int      quarter = warp & 3;         // TMEM lane quarter this warp may read
    const int      half    = (warp - 4) >> 2;  // which 128-column scale group of the tile
    const uint32_t t_lane  = ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 128);
    const uint32_t empty_leader[2] = {mapa_shared(smem_u32(&bars->part_empty[0]), 0),
                                      mapa_shared(smem_u32(&bars->part_empty[1]), 0)};
    uint32_t it = 0;
    PairWalk walk(pair, n_pairs, k_blocks, dp_tiles, split_pairs, split_s, split_chunk);
    int      tile, kb_lo, kb_hi;
    uint32_t tile_count = 0;  // SWIGLU: which exchange buffer
    // EPI_ROPE: where this warp's row quarter keeps its angle-table rows (32 rows x 512 B, 16-byte chunks
    // XOR-swizzled by row), shared by the two warps of the quarter, and the staged norm weights
    const uint32_t rope_off = EPI != EPI_ROPE ? 0u
                              : quarter == 0  ? OFF_A + (STAGES - 1) * A_BYTES
                              : quarter == 1  ? OFF_B + (STAGES - 1) * B_BYTES
                                              : OFF_STG + (quarter - 2) * ROPE_TAB_BYTES;
    const uint32_t rope_tab = smem_u32(smem + rope_off);
    const uint32_t rope_w   = smem_u32(smem + OFF_ROPE_W);
    // position of this lane's output row in tile t (rows beyond M use the first position); only the load is
    // issued here, the value is looked at a main loop later
    auto rope_row = [=](int t) -> int {
      const int mm = (t % m_tiles) * BM + (int)rank * 128 + quarter * 32 + lane;
      return __ldg(rope.pos + (mm < M ? mm : 0));
    };
    // does tile t hold a query or key head?  (the same answer in both warps of a quarter)
    auto rope_rotated = [=](int t) -> bool { return (t / m_tiles) * (BN / 128) < rope.n_q + rope.n_kv; };
    // Asynchronous copies of the quarter's 32 table rows: this warp brings the cos halves (half 0) or the sin
    // halves (half 1); one instruction moves two whole 256-byte half rows.  Nothing passes through registers and
    // nobody waits here: the rows are needed one main loop later.
    auto rope_stage = [=](int p_raw) {
      const int p_own = min(max(p_raw, 0), rope.rows - 1);
      if (p_own != p_raw) {
        atomicCAS(status, 0u, (uint32_t)DEV_BAD_POSITION);  // the access outside the tables is not made
      }
      const float* tab   = half == 0 ? rope.cos : rope.sin;
      const int    chunk = lane & 15;
#pragma unroll 4
      for (int j = 0; j < 16; ++j) {
        const int rr = 2 * j + (lane >> 4);
        const int pr = __shfl_sync(0xffffffffu, p_own, rr);
        cp_async_16(rope_tab + rr * 512 + (((half * 16 + chunk) ^ (rr & 7)) << 4), tab + (size_t)pr * 64 + chunk * 4);
      }
    };
    if constexpr (EPI == EPI_ROPE) {
      // the norm weights (ones without a weight vector: one straight line of arithmetic either way)
      const int    t    = (int)threadIdx.x - 128;
      const float* wsrc = t < 128 ? rope.q_w : rope.k_w;
      reinterpret_cast<float*>(smem + OFF_ROPE_W)[t] = wsrc != nullptr ? __ldg(wsrc + (t & 127)) : 1.0f;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (pair < dp_tiles && rope_rotated(pair)) {
        rope_stage(rope_row(pair));
      }
    }
    PROF8_STAMP(0);
    while (walk.next(tile, kb_lo, kb_hi)) {
      // EPI_ROPE: the position of this lane's row in the pair's next tile, fetched a main loop ahead of its use
      int rope_p_next = 0;
      if constexpr (EPI == EPI_ROPE) {
        if (tile + n_pairs < dp_tiles && rope_rotated(tile + n_pairs)) {
          rope_p_next = rope_row(tile + n_pairs);
        }
      }
      const int  m    = (tile % m_tiles) * BM + (int)rank * 128 + quarter * 32 + lane;
      // global 128-column group of the output (and, except for SWIGLU, of the weight scales)
      const int  ng   = SWIGLU ? tile / m_tiles : (tile / m_tiles) * (BN / 128) + half;
      const bool m_ok = m < M;
      const bool g_ok = ng < n_groups;
      const float* a_s = A_s + (m_ok ? m : 0);
      const float* b_s = B_s + (size_t)(g_ok ? ng : 0) * k_blocks;               // SWIGLU: the gate rows' scales
      const float* b_up = B_s + (size_t)(n_groups + (g_ok ? ng : 0)) * k_blocks;  // SWIGLU only: the up rows' scales

      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) {
        acc[i] = 0.0f;
      }

      // scale operands are fetched PREFETCH K-blocks ahead (an L2 hit under the TMA traffic takes
      // longer than one K-block); the empty asm pins their first use to their own iteration
      constexpr int PREFETCH = 2;
      float         a_pf[PREFETCH], b_pf[PREFETCH], b2_pf[PREFETCH];
#pragma unroll
      for (int j = 0; j < PREFETCH; ++j) {
        a_pf[j] = (kb_lo + j < kb_hi) ? __ldg(a_s + (size_t)(kb_lo + j) * M) : 0.0f;
        b_pf[j] = (kb_lo + j < kb_hi) ? __ldg(b_s + kb_lo + j) : 0.0f;
        if constexpr (SWIGLU) {
          b2_pf[j] = (kb_lo + j < kb_hi) ? __ldg(b_up + kb_lo + j) : 0.0f;
        }
      }
      for (int kb0 = kb_lo; kb0 < kb_hi; kb0 += PREFETCH) {
#pragma unroll
        for (int j = 0; j < PREFETCH; ++j) {
          const int kb = kb0 + j;
          if (kb >= kb_hi) {
            break;
          }
          const uint32_t p  = it & 1;
          const uint32_t pp = (it >> 1) & 1;
          float a_cur = a_pf[j], b_cur = b_pf[j];
          asm volatile("" : "+f"(a_cur), "+f"(b_cur));
          // one fp32 rounding of the scale product, as in the reference
          const float sc2 = __fmul_rn(a_cur, b_cur);
          float       sc2_late = sc2;  // the scale of the last 64 accumulators: the up rows' for SWIGLU
          if constexpr (SWIGLU) {
            float b2_cur = b2_pf[j];
            asm volatile("" : "+f"(b2_cur));
            sc2_late = __fmul_rn(a_cur, b2_cur);
          }
          if (kb + PREFETCH < kb_hi) {
            a_pf[j] = __ldg(a_s + (size_t)(kb + PREFETCH) * M);
            b_pf[j] = __ldg(b_s + kb + PREFETCH);
            if constexpr (SWIGLU) {
              b2_pf[j] = __ldg(b_up + kb + PREFETCH);
            }
          }
          PROF8_T(d0);
          mbar_wait(&bars->part_full[p], pp, DEV_WAIT_TMEM_FULL, abort_flag, status);
          PROF8_T(d1);
          PROF8_ADD(p_wait, d0, d1);
#ifdef LLMMM_PROFILE
          if (blockIdx.x == 0 && threadIdx.x == 128 && it < 64) {
            g_trace8[it][4] = d0;  // promotion warp 4: starts waiting for the partial
            g_trace8[it][5] = d1;  // partial observed
          }
#endif
          tc_fence_after_sync();
          const uint32_t t_addr = tmem_base + p * BN + t_lane;
          // two loads in flight; the partial stage is handed back as early as possible
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(t_addr, v0);
          tmem_ld_32x32b_x32(t_addr + 32, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            ffma2(acc[i], acc[i + 1], v0[i], v0[i + 1], sc2);
          }
          tmem_ld_32x32b_x32(t_addr + 64, v0);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            ffma2(acc[32 + i], acc[32 + i + 1], v1[i], v1[i + 1], sc2);
          }
          tmem_ld_32x32b_x32(t_addr + 96, v1);
          tmem_ld_wait();
          // every column of this thread's part of the partial stage has been read
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (rank == 0) {
              mbar_arrive(&bars->part_empty[p]);
            }
            else {
              mbar_arrive_cluster_relaxed(empty_leader[p]);
            }
          }
#ifdef LLMMM_PROFILE
          if (blockIdx.x == 0 && threadIdx.x == 128 && it < 64) {
            g_trace8[it][6] = clock64();  // partial stage handed back
          }
#endif
          // The arithmetic on the last two loads must stay behind the hand-back above: the compiler may
          // move plain FMAs across asm statements, but not asm volatile statements across one another, so
          // the scale is passed through an empty one.
          asm volatile("" : "+f"(sc2_late));
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            ffma2(acc[64 + i], acc[64 + i + 1], v0[i], v0[i + 1], sc2_late);
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            ffma2(acc[96 + i], acc[96 + i + 1], v1[i], v1[i + 1], sc2_late);
          }
          ++it;
        }
      }

      PROF8_T(e0);
      if (!SWIGLU && EPI != EPI_ROPE && kb_hi - kb_lo < k_blocks) {  // (SWIGLU and ROPE tiles are never cut)
        // A chunk of a split tile, the last piece of work of this pair.  This warp's 32x128 piece is handled
        // independently of the other warps: publish the partial sum (four columns per lane side by side:
        // a warp writes 512 contiguous bytes per instruction), count the arrival, and if it is the last
        // one for this piece, add the chunks in the order of their K ranges and finish the tile.  Nothing
        // here waits for another CTA.
        const int      tt   = tile - dp_tiles;
        const uint32_t unit = rank * 8 + (uint32_t)(warp - 4);
        float4* mine = reinterpret_cast<float4*>(sk_partials + (size_t)pair * SPLIT_SLOT_FLOATS + unit * SK_UNIT_FLOATS) + lane;
        PROF8_STAMP(1);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          __stcg(mine + i * 32, make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]));
        }
        PROF8_STAMP(2);
        __threadfence();
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) {
          arrived = atomicAdd(&sk_counters[tt * 16 + unit], 1u);
        }
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        PROF8_STAMP(4);
        if (arrived != (uint32_t)(split_s - 1)) {
          continue;  // another warp finishes this piece
        }
        __threadfence();
        if (split_s == 2) {
          // two chunks: a + b == b + a bit for bit, so this warp's own chunk can stay in its registers
          const float4* src = reinterpret_cast<const float4*>(sk_partials + (size_t)(pair ^ 1) * SPLIT_SLOT_FLOATS
                                                              + unit * SK_UNIT_FLOATS) + lane;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float4 v = __ldcg(src + i * 32);
            acc[4 * i] += v.x;
            acc[4 * i + 1] += v.y;
            acc[4 * i + 2] += v.z;
            acc[4 * i + 3] += v.w;
          }
        }
        else {
          for (int c = 0; c < split_s; ++c) {
            const float4* src = reinterpret_cast<const float4*>(sk_partials + (size_t)(tt * split_s + c) * SPLIT_SLOT_FLOATS
                                                                + unit * SK_UNIT_FLOATS) + lane;
            if (c == 0) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float4 v = __ldcg(src + i * 32);
                acc[4 * i]     = v.x;
                acc[4 * i + 1] = v.y;
                acc[4 * i + 2] = v.z;
                acc[4 * i + 3] = v.w;
              }
            }
            else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float4 v = __ldcg(src + i * 32);
                acc[4 * i] += v.x;
                acc[4 * i + 1] += v.y;
                acc[4 * i + 2] += v.z;
                acc[4 * i + 3] += v.w;
              }
            }
          }
        }
        if (lane == 0) {
          sk_counters[tt * 16 + unit] = 0;  // every launch leaves the counters at zero
        }
        PROF8_STAMP(5);
      }
      if constexpr (EPI == EPI_ROPE) {
        // ng is the head: query heads first, then key heads, then value heads (which pass unchanged).
        const int kind = ng < rope.n_q ? 0 : (ng < rope.n_q + rope.n_kv ? 1 : 2);
        if (rope_rotated(tile)) {
          // the table rows of this tile were requested a main loop ago: mine have landed, then the other warp's
          cp_async_wait_all();
          asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
          if (g_ok && kind < 2) {
            float ss4[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // four chains: a single one is 128 dependent FMAs
#pragma unroll
            for (int i = 0; i < 128; ++i) {
              ss4[i & 3] = fmaf(acc[i], acc[i], ss4[i & 3]);
            }
            const float ss = (ss4[0] + ss4[1]) + (ss4[2] + ss4[3]);
            // (the approximate instruction, 2 ulp: the exact square root and reciprocal are subroutine calls, and a
            // call here has to save accumulators on the stack)
            const bool     nrm = (kind == 0 ? rope.q_w : rope.k_w) != nullptr;
            const float    inv = nrm ? rsqrtf(fmaf(ss, 1.0f / 128.0f, rope.eps)) : 1.0f;
            const uint32_t w4  = rope_w + kind * 512;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if ((i & 3) == 0 && i > 0) {
                asm volatile("" : "+f"(acc[4 * i - 1]));  // four loads in flight at most: the next group starts here
              }
              const float4 wv = lds_pinned(w4 + i * 16);  // the same address in every lane
              acc[4 * i]      = acc[4 * i] * inv * wv.x;
              acc[4 * i + 1]  = acc[4 * i + 1] * inv * wv.y;
              acc[4 * i + 2]  = acc[4 * i + 2] * inv * wv.z;
              acc[4 * i + 3]  = acc[4 * i + 3] * inv * wv.w;
            }
            asm volatile("" : "+f"(acc[127]));  // (the rotation's loads start behind the normalisation)
            // Rotation of the half-split pairs (i, 64 + i) by the angles of this lane's own table row.
            const uint32_t row = rope_tab + lane * 512;
#pragma unroll
            for (int q4 = 0; q4 < 16; ++q4) {
              const float4 cv = lds_pinned(row + ((q4 ^ (lane & 7)) << 4));
              const float4 sn = lds_pinned(row + 256 + ((q4 ^ (lane & 7)) << 4));
              const float  cc[4] = {cv.x, cv.y, cv.z, cv.w};
              const float  sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int   i0 = 4 * q4 + e;
                const float x0 = acc[i0], x1 = acc[64 + i0];
                acc[i0]      = __fmaf_rn(x0, cc[e], -__fmul_rn(x1, sv[e]));
                acc[64 + i0] = __fmaf_rn(x1, cc[e], __fmul_rn(x0, sv[e]));
              }
              if ((q4 & 1) == 1) {
                asm volatile("" : "+f"(acc[64 + 4 * q4 + 3]));  // four loads in flight at most
              }
            }
          }
          // both warps of the quarter are done with the rows: the next tile's may be requested
          asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
        }
      }
      if constexpr (SWIGLU) {
        // acc[0..63] = gate, acc[64..127] = up of this thread's 64 output columns
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float g = acc[i];
          const float h = __fdividef(g, 1.0f + __expf(-g)) * acc[64 + i];
          acc[i]        = h;
          amax          = fmaxf(amax, fabsf(h));
        }
        // the other 64 columns of the 1x128 group belong to the thread of the same row in the other half:
        // exchange the two maxima through shared memory (two buffers, alternating from tile to tile)
        float* xch = reinterpret_cast<float*>(smem + OFF_XCH) + (tile_count & 1) * 256;
        ++tile_count;
        xch[half * 128 + quarter * 32 + lane] = amax;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        amax = fmaxf(amax, xch[(half ^ 1) * 128 + quarter * 32 + lane]);
        // The warp's 32 x 64 output bytes go through a staging tile and leave as one TMA store (whole rows instead
        // of 16-byte pieces in 32 rows per store instruction); all lanes take part, rows beyond M are clipped.
        uint8_t* stg = smem + OFF_STG_SWIGLU + (warp - 4) * 2048;
        if (lane == 0) {
          tma_store_wait_read<0>();  // the store of the previous tile has read the staging tile
        }
        __syncwarp();
        {
          const float scale     = __fdiv_rn(amax, 448.0f);
          const float scale_inv = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            o.x    = pack_e4m3x4(acc[16 * i + 0] * scale_inv, acc[16 * i + 1] * scale_inv, acc[16 * i + 2] * scale_inv, acc[16 * i + 3] * scale_inv);
            o.y    = pack_e4m3x4(acc[16 * i + 4] * scale_inv, acc[16 * i + 5] * scale_inv, acc[16 * i + 6] * scale_inv, acc[16 * i + 7] * scale_inv);
            o.z    = pack_e4m3x4(acc[16 * i + 8] * scale_inv, acc[16 * i + 9] * scale_inv, acc[16 * i + 10] * scale_inv, acc[16 * i + 11] * scale_inv);
            o.w    = pack_e4m3x4(acc[16 * i + 12] * scale_inv, acc[16 * i + 13] * scale_inv, acc[16 * i + 14] * scale_inv, acc[16 * i + 15] * scale_inv);
            *reinterpret_cast<uint4*>(stg + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4)) = o;
          }
          if (m_ok && g_ok && half == 0) {
            C_s[(size_t)ng * M + m] = scale;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && g_ok && m - lane < M) {
          tma_store_2d(&tm_c, stg, ng * 128 + half * 64, m - lane);
          tma_store_commit();
        }
      }
      else if constexpr (EPI == EPI_E4M3 || EPI == EPI_GATHER || EPI == EPI_ROPE) {
        // The whole warp takes part, also lanes of rows beyond M: the tile is transposed through shared memory.
        uint8_t* stg = smem + (EPI == EPI_ROPE ? rope_off + half * 4096 : OFF_STG + (warp - 4) * 4096);
        if constexpr (EPI == EPI_E4M3 || EPI == EPI_ROPE) {
          // the TMA store of this warp's previous tile has read the staging tile (it had a main loop's time)
          if (lane == 0) {
            tma_store_wait_read<0>();
          }
          __syncwarp();
        }
        {
          const float amax      = amax128(acc);
          const float scale     = __fdiv_rn(amax, 448.0f);
          const float scale_inv = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
          // this thread's 128 bytes go to its row of the warp's staging tile (16-byte chunks XOR-swizzled by row)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint4 o;
            o.x = pack_e4m3x4(acc[16 * i + 0] * scale_inv, acc[16 * i + 1] * scale_inv, acc[16 * i + 2] * scale_inv, acc[16 * i + 3] * scale_inv);
            o.y = pack_e4m3x4(acc[16 * i + 4] * scale_inv, acc[16 * i + 5] * scale_inv, acc[16 * i + 6] * scale_inv, acc[16 * i + 7] * scale_inv);
            o.z = pack_e4m3x4(acc[16 * i + 8] * scale_inv, acc[16 * i + 9] * scale_inv, acc[16 * i + 10] * scale_inv, acc[16 * i + 11] * scale_inv);
            o.w = pack_e4m3x4(acc[16 * i + 12] * scale_inv, acc[16 * i + 13] * scale_inv, acc[16 * i + 14] * scale_inv, acc[16 * i + 15] * scale_inv);
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((i ^ (lane & 7)) << 4)) = o;
          }
          if (m_ok && g_ok) {  // 32 consecutive floats per warp
            if constexpr (EPI == EPI_GATHER) {
              const size_t s_off = (size_t)(gather.col0 / 128 + ng) * M + m;
              for (int d = 0; d < gather.n; ++d) {
                gather.cs[d][s_off] = scale;
              }
            }
            else {
              C_s[(size_t)ng * M + m] = scale;
            }
          }
        }
        if constexpr (EPI == EPI_E4M3 || EPI == EPI_ROPE) {
          // one asynchronous store of the whole 32 x 128-byte tile; rows beyond M are clipped by the tensor map
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && g_ok && m - lane < M) {
            tma_store_2d(&tm_c, stg, ng * 128, m - lane);
            tma_store_commit();
          }
        }
        else {
        __syncwarp();
        // one store instruction now covers four whole rows: lane l writes chunk l & 7 of row 4 i + (l >> 3)
        // (for EPI_GATHER: what crosses to the other GPUs are contiguous 128-byte rows, not 16-byte pieces)
        if (g_ok) {
          const int    m_warp = m - lane;
          const size_t col    = (size_t)(EPI == EPI_GATHER ? gather.col0 : 0) + (size_t)ng * 128 + (size_t)((lane & 7) << 4);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int   rr = 4 * i + (lane >> 3);
            const uint4 o  = *reinterpret_cast<const uint4*>(stg + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
            if (m_warp + rr < M) {
              if constexpr (EPI == EPI_GATHER) {
                for (int d = 0; d < gather.n; ++d) {
                  *reinterpret_cast<uint4*>(gather.c[d] + (size_t)(m_warp + rr) * gather.ld + col) = o;
                }
              }
              else {
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(C_out) + (size_t)(m_warp + rr) * N + col) = o;
              }
            }
          }
        }
        __syncwarp();
        }
      }
      else if constexpr (OUT_F32) {
        // A thread's row of the tile is 512 bytes; written directly, every store instruction would touch 32 rows.
        // Four passes of 32 columns each through the warp's staging tile instead, each leaving as one TMA store
        // (the tensor map sees C as [M, 4 N] bytes).  The whole warp takes part; rows beyond M are clipped.
        uint8_t* stg = smem + OFF_STG + (warp - 4) * 4096;
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {
          if (lane == 0) {
            tma_store_wait_read<0>();  // the previous store has read the staging tile
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            *reinterpret_cast<float4*>(stg + lane * 128 + ((i ^ (lane & 7)) << 4)) =
              make_float4(acc[32 * ps + 4 * i], acc[32 * ps + 4 * i + 1], acc[32 * ps + 4 * i + 2], acc[32 * ps + 4 * i + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && g_ok && m - lane < M) {
            tma_store_2d(&tm_c, stg, ng * 512 + ps * 128, m - lane);
            tma_store_commit();
          }
        }
      }
      else {
        static_assert(EPI == EPI_SWIGLU, "every other epilogue is handled above");
      }
      if constexpr (EPI == EPI_ROPE) {
        if (tile + n_pairs < dp_tiles && rope_rotated(tile + n_pairs)) {
          // (the stores of both warps of the quarter have read their staging tiles, which lie in the region the
          // rows go to)
          if (lane == 0) {
            tma_store_wait_read<0>();
          }
          asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
          rope_stage(rope_p_next);
        }
      }
      PROF8_T(e1);
      PROF8_ADD(p_epi, e0, e1);
      if (kb_hi - kb_lo < k_blocks) {
        PROF8_STAMP(6);
      }
    }
    if constexpr (EPI != EPI_GATHER) {
      if (lane == 0) {
        tma_store_wait_read<0>();  // shared memory must outlive the last store's read of it
      }
    }
#ifdef LLMMM_PROFILE
    if (blockIdx.x == 0 && threadIdx.x == 128) {
      g_prof8[8]  = clock64() - p_p0;
      g_prof8[9]  = p_wait;
      g_prof8[10] = p_epi;
      g_prof8[11] = it;
    }
#endif
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

template<int EPI>
static int launch_fp8_pair_epi(const void*       A,
                               const float*      A_s,
                               const void*       B,
                               const float*      B_s,
                               void*             C,
                               float*            C_s,
                               int               M,
                               int               N,
                               int               K,
                               const RopeHook&   hook,
                               const DeviceInfo* info,
                               cudaStream_t      stream)
{
  using namespace fp8pair;
  CUtensorMap tm_a, tm_b;
  if (!make_tmap_2d(&tm_a, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_b, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  CUtensorMap tm_c = {};
  if constexpr (EPI == EPI_E4M3 || EPI == EPI_ROPE || EPI == EPI_F32) {
    const uint64_t row_bytes = (uint64_t)N * (EPI == EPI_F32 ? 4 : 1);
    if (!make_tmap_2d(&tm_c, C, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, row_bytes, (uint64_t)M, row_bytes, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
      return LLMMM_ERR_CUDA;
    }
  }
  constexpr uint32_t SMEM = smem_bytes_of(EPI);
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(cudaFuncSetAttribute(
      fp8_blockwise_gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    attr_set[info->device] = true;
  }
  const int tiles    = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int k_blocks = K / BK;
  // estimated cost of a split, in K-blocks (one takes about 0.58 us): publishing a chunk and counting the
  // arrival about 3 us, reading a chunk back about 1.5 us
  SplitPlan plan = plan_split(info, tiles, k_blocks, /*fixed*/ 4, /*per_way_x2*/ 5, /*min_gain*/ 3, /*count*/ EPI != EPI_ROPE);
  if constexpr (EPI == EPI_ROPE) {
    // whole tiles only: this instantiation has no code for the chunks of a cut tile (no register left for it)
    plan = SplitPlan{tiles, 0, 1, k_blocks, tiles < info->max_pairs ? tiles : info->max_pairs, nullptr, nullptr};
  }
  LLMMM_CUDA_TRY(launch_pdl(fp8_blockwise_gemm_pair_kernel<EPI>, dim3(2 * plan.pairs), dim3(THREADS), SMEM, stream,
                            2, tm_a, tm_b, tm_c, A_s, B_s, C, C_s, M, N, K, plan.dp_tiles, plan.split_pairs, plan.split_s,
                            plan.split_chunk, plan.partials, plan.counters, GatherDst{}, hook, info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

template<bool OUT_F32>
static int launch_fp8_pair(const void* A, const float* A_s, const void* B, const float* B_s, void* C, float* C_s, int M,
                           int N, int K, const DeviceInfo* info, cudaStream_t stream)
{
  return launch_fp8_pair_epi<(OUT_F32 ? EPI_F32 : EPI_E4M3)>(A, A_s, B, B_s, C, C_s, M, N, K, RopeHook{}, info, stream);
}

// gate_up GEMM with the SwiGLU epilogue: B [2I, K], B_s [2I/128, K/128], H_q [M, I], H_s [I/128, M].
static int launch_fp8_swiglu(const void*       A,
                             const float*      A_s,
                             const void*       B,
                             const float*      B_s,
                             void*             H,
                             float*            H_s,
                             int               M,
                             int               I,
                             int               K,
                             const DeviceInfo* info,
                             cudaStream_t      stream)
{
  using namespace fp8pair;
  CUtensorMap tm_a, tm_b;
  if (!make_tmap_2d(&tm_a, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_b, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)2 * I, (uint64_t)K, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  CUtensorMap tm_h;  // H as [M, I] bytes, boxes of 32 rows x 64 bytes
  if (!make_tmap_2d(&tm_h, H, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)I, (uint64_t)M, (uint64_t)I, 64, 32, CU_TENSOR_MAP_SWIZZLE_64B)) {
    return LLMMM_ERR_CUDA;
  }
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(cudaFuncSetAttribute(
      fp8_blockwise_gemm_pair_kernel<EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES_SWIGLU));
    attr_set[info->device] = true;
  }
  // a tile is 256 rows x 128 output columns (128 gate + 128 up weight rows); tiles are never cut along K here:
  // the two threads that share a 1x128 output group would have to finish the same piece
  const int tiles = ((M + BM - 1) / BM) * (I / 128);
  const int pairs = tiles < info->max_pairs ? tiles : info->max_pairs;
  float*    no_partials = nullptr;
  uint32_t* no_counters = nullptr;
  LLMMM_CUDA_TRY(launch_pdl(fp8_blockwise_gemm_pair_kernel<EPI_SWIGLU>, dim3(2 * pairs), dim3(THREADS), SMEM_BYTES_SWIGLU, stream, 2,
                            tm_a, tm_b, tm_h, A_s, B_s, H, H_s, M, I, K, tiles, 0, 1, K / BK, no_partials, no_counters,
                            GatherDst{}, RopeHook{}, info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

// Column shard [col0, col0 + N) of a wider product, stored into every destination's full C (EPI_GATHER).
static int launch_fp8_gather(const void*       A,
                             const float*      A_s,
                             const void*       B,
                             const float*      B_s,
                             const GatherDst&  dst,
                             int               M,
                             int               N,
                             int               K,
                             const DeviceInfo* info,
                             cudaStream_t      stream)
{
  using namespace fp8pair;
  CUtensorMap tm_a, tm_b;
  if (!make_tmap_2d(&tm_a, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_b, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(cudaFuncSetAttribute(
      fp8_blockwise_gemm_pair_kernel<EPI_GATHER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES_STAGED));
    attr_set[info->device] = true;
  }
  const int       tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const SplitPlan plan  = plan_split(info, tiles, K / BK, /*fixed*/ 4, /*per_way_x2*/ 5, /*min_gain*/ 3);
  float*          none  = nullptr;
  LLMMM_CUDA_TRY(launch_pdl(fp8_blockwise_gemm_pair_kernel<EPI_GATHER>, dim3(2 * plan.pairs), dim3(THREADS), SMEM_BYTES_STAGED, stream, 2,
                            tm_a, tm_b, CUtensorMap{}, A_s, B_s, static_cast<void*>(nullptr), none, M, N, K, plan.dp_tiles, plan.split_pairs,
                            plan.split_s, plan.split_chunk, plan.partials, plan.counters, dst, RopeHook{}, info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
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
  if (fp8_use_pair_kernel(info, M, N, K)) {
    return launch_fp8_pair<OUT_F32>(A, A_s, B, B_s, C, C_s, M, N, K, info, stream);
  }
  CUtensorMap tm_a, tm_b;
  if (!make_tmap_2d(&tm_a, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_b, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  CUtensorMap tm_c = {};  // the e4m3 output as [M, N] bytes, boxes of 32 rows x 128 bytes
  if (!OUT_F32 && !make_tmap_2d(&tm_c, C, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)M, (uint64_t)N, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
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
  LLMMM_CUDA_TRY(launch_pdl(fp8_blockwise_gemm_kernel<OUT_F32>, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, 1, tm_a, tm_b,
                            tm_c, A_s, B_s, C, C_s, M, N, K, info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

void describe_fp8_plan(const DeviceInfo* info, bool out_f32, int M, int N, int K, char* buf, size_t len)
{
  const char* o = out_f32 ? "true" : "false";
  if (describe_decode_plan(info, M, N, K, buf, len)) {
    return;
  }
  bool        tuned = false;
  const bool  pair  = fp8_use_pair_kernel(info, M, N, K, &tuned);
  const char* how   = (M > 64 && M <= 128) ? (tuned ? " (kernel choice: measured by llmmm_tune)" : " (kernel choice: default rule)") : "";
  if (pair) {
    using namespace fp8pair;
    const int       tiles    = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int       k_blocks = K / BK;
    const SplitPlan plan     = plan_split(info, tiles, k_blocks, 4, 5, 3, false);
    if (plan.split_pairs > 0) {
      snprintf(buf, len, "fp8_blockwise_gemm_pair_kernel<%s>: %d tiles of 256x256 on %d CTA pairs; %d whole tiles round-robin, then "
               "%d tiles cut %d-way along K (chunks of %d K-blocks), one chunk per pair%s", o, tiles, plan.pairs, plan.dp_tiles,
               tiles - plan.dp_tiles, plan.split_s, plan.split_chunk, how);
    }
    else {
      snprintf(buf, len, "fp8_blockwise_gemm_pair_kernel<%s>: %d tiles of 256x256 on %d CTA pairs (%.2f waves), %d K-blocks each, "
               "no split%s", o, tiles, plan.pairs, (double)tiles / plan.pairs, k_blocks, how);
    }
    return;
  }
  using namespace fp8cfg;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid  = tiles < info->sm_count ? tiles : info->sm_count;
  snprintf(buf, len, "fp8_blockwise_gemm_kernel<%s>: %d tiles of %dx%d on %d CTAs (%.2f waves)%s", o, tiles, BM, BN, grid,
           (double)tiles / grid, how);
}

int launch_fp8_e4m3(const void* A, const float* A_s, const void* B, const float* B_s, void* C, float* C_s, int M, int N, int K,
                    cudaStream_t stream)
{
  return launch_fp8<false>(A, A_s, B, B_s, C, C_s, M, N, K, stream);
}

int warm_fp8_kernels(const DeviceInfo* info)
{
  (void)info;
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_blockwise_gemm_pair_kernel<EPI_E4M3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp8pair::SMEM_BYTES_STAGED));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_blockwise_gemm_pair_kernel<EPI_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp8pair::SMEM_BYTES_STAGED));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_blockwise_gemm_pair_kernel<EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp8pair::SMEM_BYTES_SWIGLU));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_blockwise_gemm_pair_kernel<EPI_GATHER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp8pair::SMEM_BYTES_STAGED));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_blockwise_gemm_pair_kernel<EPI_ROPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp8pair::SMEM_BYTES_ROPE));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_blockwise_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp8cfg::SMEM_BYTES));
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_blockwise_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp8cfg::SMEM_BYTES));
  return warm_decode_kernels(info);
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

#ifdef LLMMM_PROFILE
extern "C" void llmmm_profile_trace8()
{
  long long t[64][8];
  cudaMemcpyFromSymbol(t, llmmm::g_trace8, sizeof(t));
  const long long t0 = t[8][0];
  printf("K-block: MMA[wait_part free operands issued] PROMO[wait observed released]  (clk relative)\n");
  for (int i = 8; i < 24; ++i) {
    printf("%2d: %6lld %6lld %6lld %6lld | %6lld %6lld %6lld\n", i, t[i][0] - t0, t[i][1] - t0, t[i][2] - t0, t[i][3] - t0,
           t[i][4] - t0, t[i][5] - t0, t[i][6] - t0);
  }
}

extern "C" void llmmm_profile_stamps8()
{
  unsigned long long t[4][16];
  cudaMemcpyFromSymbol(t, llmmm::g_stamp8, sizeof(t));
  for (int b = 0; b < 4; ++b) {
    printf("CTA %d warp 4 (ns from start of its role): chunk done %lld, published %lld, all work done %lld, arrival counted %lld, "
           "chunks summed %lld, epilogue done %lld\n", b, (long long)(t[b][1] - t[b][0]), (long long)(t[b][2] - t[b][0]),
           (long long)(t[b][3] - t[b][0]), (long long)(t[b][4] - t[b][0]), (long long)(t[b][5] - t[b][0]),
           (long long)(t[b][6] - t[b][0]));
  }
}

extern "C" void llmmm_profile_dump8()
{
  long long h[16];
  cudaMemcpyFromSymbol(h, llmmm::g_prof8, sizeof(h));
  printf("fp8 pair kernel CTA 0: %.3f GHz, %.1f us, %lld K-blocks, %.0f clk/K-block; MMA thread waits: operands %.0f, "
         "free partial %.0f clk/K-block; promotion warp 4: total %.0f, waiting for partials %.0f, epilogue %.0f clk/K-block\n",
         (double)h[0] / h[1], h[1] / 1e3, h[4], (double)h[0] / h[4], (double)h[2] / h[4], (double)h[3] / h[4],
         (double)h[8] / h[11], (double)h[9] / h[11], (double)h[10] / h[11]);
}
#endif

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

int llmmm_fp8_blockwise_mm_e4m3out_ws(const void*    A,
                                      const float*   A_scale_t,
                                      const void*    B_t,
                                      const float*   B_scale_t,
                                      void*          C,
                                      float*         C_scale_t,
                                      int            M,
                                      int            N,
                                      int            K,
                                      void*          workspace,
                                      size_t         workspace_bytes,
                                      llmmm_stream_t stream)
{
  const int rc = llmmm::check_workspace_arg(workspace, workspace_bytes);
  if (rc != LLMMM_OK) {
    return rc;
  }
  llmmm::ScopedWorkspace bound(workspace, workspace_bytes);  // this call sees `workspace`, whatever is registered
  return llmmm_fp8_blockwise_mm_e4m3out(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K, stream);
}

int llmmm_fp8_blockwise_mm_f32out_ws(const void*    A,
                                     const float*   A_scale_t,
                                     const void*    B_t,
                                     const float*   B_scale_t,
                                     float*         C,
                                     int            M,
                                     int            N,
                                     int            K,
                                     void*          workspace,
                                     size_t         workspace_bytes,
                                     llmmm_stream_t stream)
{
  const int rc = llmmm::check_workspace_arg(workspace, workspace_bytes);
  if (rc != LLMMM_OK) {
    return rc;
  }
  llmmm::ScopedWorkspace bound(workspace, workspace_bytes);
  return llmmm_fp8_blockwise_mm_f32out(A, A_scale_t, B_t, B_scale_t, C, M, N, K, stream);
}

int llmmm_fp8_blockwise_mm_e4m3out_gather(const void*    A,
                                          const float*   A_scale_t,
                                          const void*    B_t,
                                          const float*   B_scale_t,
                                          void* const*   C_dsts,
                                          float* const*  C_scale_dsts,
                                          int            n_dsts,
                                          int            N_total,
                                          int            col_offset,
                                          int            M,
                                          int            N,
                                          int            K,
                                          llmmm_stream_t stream)
{
  using namespace llmmm;
  int rc = check_fp8_args(A, A_scale_t, B_t, B_scale_t, A, M, N, K);
  if (rc != LLMMM_OK) {
    return rc;
  }
  if (C_dsts == nullptr || C_scale_dsts == nullptr || n_dsts < 1 || n_dsts > 8) {
    return set_error(LLMMM_ERR_SHAPE, "between 1 and 8 destinations are needed (got %d)", n_dsts);
  }
  if ((N_total % 128) != 0 || (col_offset % 128) != 0 || col_offset < 0 || col_offset + N > N_total) {
    return set_error(LLMMM_ERR_SHAPE, "the shard [%d, %d) must lie on 128-column boundaries inside the %d columns of C",
                     col_offset, col_offset + N, N_total);
  }
  GatherDst dst{};
  for (int d = 0; d < n_dsts; ++d) {
    if (C_dsts[d] == nullptr || C_scale_dsts[d] == nullptr || ((uintptr_t)C_dsts[d] & 15)) {
      return set_error(LLMMM_ERR_SHAPE, "destination %d: null or not 16-byte aligned", d);
    }
    dst.c[d]  = static_cast<uint8_t*>(C_dsts[d]);
    dst.cs[d] = C_scale_dsts[d];
  }
  dst.n    = n_dsts;
  dst.ld   = N_total;
  dst.col0 = col_offset;
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  if (info->max_pairs < 1) {
    return set_error(LLMMM_ERR_UNSUPPORTED, "this device cannot hold a cluster of two CTAs of the GEMM kernel");
  }
  return launch_fp8_gather(A, A_scale_t, B_t, B_scale_t, dst, M, N, K, info, reinterpret_cast<cudaStream_t>(stream));
}

int llmmm_fp8_blockwise_mm_swiglu_e4m3out(const void*    A,
                                          const float*   A_scale_t,
                                          const void*    B_gate_up_t,
                                          const float*   B_scale_t,
                                          void*          H,
                                          float*         H_scale_t,
                                          int            M,
                                          int            I,
                                          int            K,
                                          llmmm_stream_t stream)
{
  using namespace llmmm;
  if (A == nullptr || A_scale_t == nullptr || B_gate_up_t == nullptr || B_scale_t == nullptr || H == nullptr
      || H_scale_t == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (M < 1 || I < 128 || K < 128 || (I % 128) != 0 || (K % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "M or I or K are not aligned. (need M>=1, I%%128==0, K%%128==0; got %d %d %d)", M, I, K);
  }
  if (((uintptr_t)A | (uintptr_t)B_gate_up_t | (uintptr_t)H) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "A, B and H must be 16-byte aligned");
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (M <= 64) {
    // Decode-sized: the weight-streaming decode kernel leaves the [M, 2I] accumulator in the registered scratch
    // (behind its own partial tiles) and a second, tiny kernel applies SwiGLU and quantises.  Without enough
    // scratch the 256-row kernel below runs (correct, but it reads the weights at a fraction of the rate).
    const Workspace ws  = registered_workspace(info->device);
    const size_t    off = (decode_workspace_bytes(M) + 255) & ~size_t(255);
    if (ws.ptr != nullptr && ws.bytes >= off + (size_t)M * 2 * I * sizeof(float)) {
      float*    acc = reinterpret_cast<float*>(static_cast<uint8_t*>(ws.ptr) + off);
      const int rc  = launch_decode(true, A, A_scale_t, B_gate_up_t, B_scale_t, acc, nullptr, M, 2 * I, K, s);
      if (rc == LLMMM_OK) {
        return launch_swiglu_quant(acc, H, H_scale_t, M, I, s);
      }
      if (rc > 0) {
        return rc;
      }
    }
  }
  if (info->max_pairs < 1) {
    return set_error(LLMMM_ERR_UNSUPPORTED, "this device cannot hold a cluster of two CTAs of the GEMM kernel");
  }
  return launch_fp8_swiglu(A, A_scale_t, B_gate_up_t, B_scale_t, H, H_scale_t, M, I, K, info, s);
}

int llmmm_fp8_blockwise_mm_qk_norm_rope_e4m3out(const void*    A,
                                                const float*   A_scale_t,
                                                const void*    B_t,
                                                const float*   B_scale_t,
                                                void*          C,
                                                float*         C_scale_t,
                                                const int*     positions,
                                                const float*   cos_table,
                                                const float*   sin_table,
                                                int            table_rows,
                                                const float*   q_norm_weight,
                                                const float*   k_norm_weight,
                                                float          eps,
                                                int            n_q_heads,
                                                int            n_kv_heads,
                                                int            M,
                                                int            N,
                                                int            K,
                                                llmmm_stream_t stream)
{
  using namespace llmmm;
  if (A == nullptr || A_scale_t == nullptr || B_t == nullptr || B_scale_t == nullptr || C == nullptr || C_scale_t == nullptr
      || positions == nullptr || cos_table == nullptr || sin_table == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (M < 1 || N < 128 || K < 128 || (N % 128) != 0 || (K % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "M or N or K are not aligned. (need M>=1, N%%128==0, K%%128==0; got %d %d %d)", M, N, K);
  }
  if (n_q_heads < 0 || n_kv_heads < 0 || (long long)(n_q_heads + 2LL * n_kv_heads) * 128 != N) {
    return set_error(LLMMM_ERR_SHAPE, "N must be (n_q_heads + 2 n_kv_heads) * 128 (got N=%d, %d query and %d key/value heads)", N,
                     n_q_heads, n_kv_heads);
  }
  if (((uintptr_t)A | (uintptr_t)B_t | (uintptr_t)C | (uintptr_t)cos_table | (uintptr_t)sin_table | (uintptr_t)q_norm_weight
       | (uintptr_t)k_norm_weight)
      & 15) {
    return set_error(LLMMM_ERR_SHAPE, "A, B, C, the angle tables and the norm weights must be 16-byte aligned");
  }
  if (!(eps >= 0.0f)) {
    return set_error(LLMMM_ERR_SHAPE, "eps must be non-negative");
  }
  if (table_rows < 1) {
    return set_error(LLMMM_ERR_SHAPE, "the angle tables need at least one row (got table_rows=%d)", table_rows);
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  const RopeHook hook{cos_table, sin_table, positions, q_norm_weight, k_norm_weight, eps, n_q_heads, n_kv_heads, table_rows};
  cudaStream_t   s = reinterpret_cast<cudaStream_t>(stream);
  if (M <= 64) {
    // Decode-sized: the weight-streaming decode kernel leaves the [M, N] accumulator in the registered scratch
    // (behind its own partial tiles) and a second, tiny kernel applies the hook and quantises.  Without enough
    // scratch the 256-row kernel below runs (correct, but it reads the weights at a fraction of the rate).
    const Workspace ws  = registered_workspace(info->device);
    const size_t    off = (decode_workspace_bytes(M) + 255) & ~size_t(255);
    if (ws.ptr != nullptr && ws.bytes >= off + (size_t)M * N * sizeof(float)) {
      float*    acc = reinterpret_cast<float*>(static_cast<uint8_t*>(ws.ptr) + off);
      const int rc  = launch_decode(true, A, A_scale_t, B_t, B_scale_t, acc, nullptr, M, N, K, s);
      if (rc == LLMMM_OK) {
        return launch_rope_quant(acc, C, C_scale_t, hook, M, N, info->status, s);
      }
      if (rc > 0) {
        return rc;
      }
    }
  }
  if (info->max_pairs < 1) {
    return set_error(LLMMM_ERR_UNSUPPORTED, "this device cannot hold a cluster of two CTAs of the GEMM kernel");
  }
  return launch_fp8_pair_epi<EPI_ROPE>(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K, hook, info, s);
}

size_t llmmm_fp8_qk_norm_rope_workspace_bytes(int M, int N, int K)
{
  if (M < 1 || N < 128) {
    return 0;
  }
  (void)K;
  if (M > 64) {
    return 0;  // the fused kernel runs whole tiles and needs no scratch
  }
  return ((llmmm::decode_workspace_bytes(M) + 255) & ~size_t(255)) + (size_t)M * N * sizeof(float);
}

size_t llmmm_fp8_swiglu_workspace_bytes(int M, int I, int K)
{
  (void)K;
  if (M < 1 || M > 64 || I < 128) {
    return 0;  // larger M: the fused kernel needs no scratch
  }
  return ((llmmm::decode_workspace_bytes(M) + 255) & ~size_t(255)) + (size_t)M * 2 * I * sizeof(float);
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
