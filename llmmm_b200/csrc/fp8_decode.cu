// Decode-sized (M <= 64) FP8 e4m3 blockwise GEMM for sm_100a: the weight
// stream is the whole cost, so the kernel is organised around HBM bandwidth.
//
// Same arithmetic contract as fp8_mm.cu (reference kernels
// examples/005.fp8.mm.cu:565-2464, which cannot run M < 128 at all and have no
// split-K, README.md:22).  Organisation:
//
//   * swap-AB: a 128x128-byte weight block B_q[nb*128.., kb*128..] is the
//     128-row operand of tcgen05.mma.kind::f8f6f4 and the (zero-padded)
//     activation rows are the narrow N side (16, 32 or 64 columns), so TMEM
//     lane = output column n and TMEM column = output row m;
//   * stream-K: the (N/128 x K/128) grid of weight blocks is cut into one
//     contiguous run per CTA, so all SMs stream the same number of bytes
//     whatever N is; a run crosses output groups, giving "segments";
//   * warp 0 streams weight blocks (and the matching activation slab) through
//     an 8-deep TMA ring, warp 1 issues four MMAs per K-block from zero into
//     one of two TMEM partial stages, warps 2-5 promote with
//     acc = fma(partial, A_s*B_s, acc) in registers;
//   * a segment that covers a group's whole K range is finished in place;
//     otherwise its fp32 partial goes to the caller's scratch buffer and the
//     last CTA to arrive at the group's counter (no CTA ever waits for another)
//     adds the partials in fixed CTA order, so results do not depend on timing;
//   * the 1x128 output group runs across the 128 lanes in this orientation:
//     the group absmax is a warp-shuffle reduction plus a 4-entry exchange in
//     shared memory between the four warps.
#include <cuda_fp8.h>
#include <mutex>

#include "host_common.h"
#include "sm100.cuh"

namespace llmmm {

namespace deccfg {
constexpr int      BK            = 128;
constexpr int      UMMA_K        = 32;
constexpr int      MAX_STAGES    = 6;    // the ring depth depends on the activation tile, see DecodeSmem
constexpr int      THREADS       = 192;
constexpr uint32_t W_BYTES       = 128 * BK;
constexpr int      MAX_CTAS      = 256;
constexpr int      MAX_GROUPS    = 4096;                 // counters: N <= 524288
constexpr size_t   COUNTER_BYTES = MAX_GROUPS * sizeof(uint32_t);
constexpr uint32_t TMEM_COLS     = 256;  // one partial stage per ring stage (see DecodeSmem), two CTAs per SM
}  // namespace deccfg

template<int MP>
struct DecodeSmem {
  static constexpr uint32_t X_BYTES    = MP * deccfg::BK;
  // As deep a ring as lets two CTAs share an SM (113 KB each; tensor memory: 256 columns each): the next
  // kernel of a launch chain then sets up, and requests static weights, beside the running one.
  static constexpr int      STAGES     = MP <= 16 ? 6 : (MP <= 32 ? 5 : 4);
  // K-block `it` uses ring stage it % STAGES and the tensor-memory partial stage of the same index, so ONE
  // tcgen05.commit per K-block tells both the promotion warps (partial ready) and the producer (operands
  // consumed); a second commit would cost the single issuing thread another ~150 clk per K-block.
  static constexpr uint32_t PART_COLS  = MP < 32 ? 32 : MP;
  static_assert(STAGES * PART_COLS <= deccfg::TMEM_COLS, "partial stages exceed the tensor memory allocation");
  static constexpr uint32_t OFF_W      = 0;
  static constexpr uint32_t OFF_X      = STAGES * deccfg::W_BYTES;
  static constexpr uint32_t OFF_BAR    = OFF_X + STAGES * X_BYTES;
  // at least 80 KB, so that never more than two CTAs share an SM: a third one would sit in tcgen05.alloc until
  // tensor memory is freed
  static constexpr uint32_t USED_BYTES = OFF_BAR + 2048 + 1024;
  static constexpr uint32_t SMEM_BYTES = USED_BYTES > 80 * 1024 ? USED_BYTES : 80 * 1024;
};

struct DecodeBars {
  uint64_t full[deccfg::MAX_STAGES];        // operands of the stage have landed
  uint64_t part_full[deccfg::MAX_STAGES];   // the K-block's MMAs are done: partial ready, operands consumed
  uint64_t part_empty[deccfg::MAX_STAGES];  // the 4 promotion warps have copied the partial out
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t last_flag;
  uint32_t pad;
  float    amax[4][64];
  float    inv[64];
};

#ifdef LLMMM_PROFILE
// Debug build only: %globaltimer at the phases of CTA 0 (see llmmm_profile_dump_decode()).
__device__ unsigned long long g_prof_dec[16];
__device__ unsigned long long g_prof_cta[256][4];  // per CTA: entry, promotion loop done, fix-up done, exit
__device__ unsigned long long g_prof_fin[256][6];  // last segment: published, counted, reduced, amax, stored
__device__ unsigned long long g_prof_pdl[256][2];  // producer thread: before / after waiting for the previous kernel
__device__ unsigned long long g_prof_set[256][4];  // set-up: barriers initialised, before / after tcgen05.alloc, after the CTA barrier
#define PROFF(i) if (et == 0) g_prof_fin[blockIdx.x][i] = global_timer_ns()
#else
#define PROFF(i)
#endif
#ifdef LLMMM_PROFILE
#define PROFD(i) if (blockIdx.x == 0) g_prof_dec[i] = global_timer_ns()
#else
#define PROFD(i)
#endif

__device__ __forceinline__ void epilogue_bar_sync()
{
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// unit u of the (group, K-block) grid belongs to CTA ((u+1)*G - 1) / U, the
// largest c with floor(c*U/G) <= u.
__device__ __forceinline__ int cta_of_unit(uint32_t u, uint32_t G, uint32_t U)
{
  return (int)(((u + 1) * G - 1) / U);
}

// CLUSTER = false: stream-K over all weight blocks, partial tiles through the caller's scratch (above).
// CLUSTER = true : one thread-block cluster per output group; CTA r of the C in the cluster takes the r-th
//   slice of the group's K range, and the partial tiles are added through distributed shared memory: after
//   a cluster barrier (every CTA's TMA ring is idle) the other CTAs store their partial into the leader's
//   ring, a second barrier, and the leader adds them in rank order and runs the epilogue.  No scratch, no
//   atomics, no global round trips; used when the groups times a cluster size of 2-7 fill the GPU.
template<int MP, bool OUT_F32, bool CLUSTER>
__global__ void __launch_bounds__(deccfg::THREADS, 2) fp8_decode_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                        const __grid_constant__ CUtensorMap tm_x,
                                                                        const float* __restrict__ A_s,
                                                                        const float* __restrict__ B_s,
                                                                        void* __restrict__ C_out,
                                                                        float* __restrict__ C_s,
                                                                        int       M,
                                                                        int       N,
                                                                        int       K,
                                                                        float*    partials,
                                                                        uint32_t* counters,
                                                                        int       early_weights,
                                                                        uint32_t* status)
{
  using namespace deccfg;
  using L = DecodeSmem<MP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t*    smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  DecodeBars* bars = reinterpret_cast<DecodeBars*>(smem + L::OFF_BAR);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    PROFD(0);
#ifdef LLMMM_PROFILE
    g_prof_cta[blockIdx.x][0] = global_timer_ns();
#endif
  }

  const int       KB      = K / BK;
  const uint32_t  U       = (uint32_t)(N / 128) * (uint32_t)KB;  // the launcher keeps U * 256 below 2^31
  const uint32_t  G       = gridDim.x;
  uint32_t        c_size  = 1, c_rank = 0;
  uint32_t        u_begin, u_end;
  if constexpr (CLUSTER) {
    asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(c_size));
    c_rank = cluster_ctarank();
    const uint32_t group = blockIdx.x / c_size;
    u_begin = group * (uint32_t)KB + (c_rank * (uint32_t)KB) / c_size;
    u_end   = group * (uint32_t)KB + ((c_rank + 1) * (uint32_t)KB) / c_size;
  }
  else {
    u_begin = (blockIdx.x * U) / G;
    u_end   = ((blockIdx.x + 1) * U) / G;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->part_full[s], 1);
      mbar_init(&bars->part_empty[s], 4);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
#ifdef LLMMM_PROFILE
    g_prof_set[blockIdx.x][0] = global_timer_ns();
#endif
  }
  if (warp == 1) {
#ifdef LLMMM_PROFILE
    if (lane == 0) g_prof_set[blockIdx.x][1] = global_timer_ns();
#endif
    tmem_alloc<TMEM_COLS>(&bars->tmem_base);
#ifdef LLMMM_PROFILE
    if (lane == 0) g_prof_set[blockIdx.x][2] = global_timer_ns();
#endif
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
#ifdef LLMMM_PROFILE
  if (threadIdx.x == 0) g_prof_set[blockIdx.x][3] = global_timer_ns();
#endif
  const uint32_t tmem_base = bars->tmem_base;
  // Set-up (barriers, tensor memory, descriptor prefetch) touched no global memory: it may overlap the tail
  // of the previous kernel on the stream, and the next kernel may begin its own set-up from here on.
  pdl_launch_dependents();
  if (warp != 0) {
    pdl_wait();  // warp 0 waits below, as a whole: a waiting lane holds up the other lanes of its warp
  }
  if (threadIdx.x == 0) {
    PROFD(1);
  }

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    const uint64_t pol_w = policy_evict_first();  // weights are read once
    const uint64_t pol_x = policy_evict_last();   // activations are re-read by every CTA
    const int      nb0   = (int)(u_begin / (uint32_t)KB);
    const int      kb0   = (int)(u_begin % (uint32_t)KB);
    // Weights the caller declared static (llmmm_set_static_weights) do not depend on the previous kernel
    // of the stream: the first ring of weight tiles is requested before waiting for that kernel, the
    // activation tiles of the same stages after it.
    uint32_t early = 0;
    if (lane == 0 && early_weights) {
      int nb = nb0, kb = kb0;
      for (uint32_t u = u_begin; u < u_end && early < (uint32_t)L::STAGES; ++u, ++early, ++kb) {
        if (kb == KB) {
          kb = 0;
          ++nb;
        }
        mbar_arrive_expect_tx(&bars->full[early], W_BYTES + L::X_BYTES);
        tma_load_2d_hint(smem + L::OFF_W + early * W_BYTES, &tm_w, &bars->full[early], kb * BK, nb * 128, pol_w);
      }
    }
    __syncwarp();
#ifdef LLMMM_PROFILE
    if (lane == 0) g_prof_pdl[blockIdx.x][0] = global_timer_ns();
#endif
    pdl_wait();
#ifdef LLMMM_PROFILE
    if (lane == 0) g_prof_pdl[blockIdx.x][1] = global_timer_ns();
#endif
    if (lane == 0) {
      uint32_t it = 0;
      int      nb = nb0, kb = kb0;
      for (uint32_t u = u_begin; u < u_end; ++u, ++it, ++kb) {
        if (kb == KB) {
          kb = 0;
          ++nb;
        }
        const uint32_t s  = it % L::STAGES;
        const uint32_t ph = (it / L::STAGES) & 1;
        if (it >= early) {
          mbar_wait(&bars->part_full[s], ph ^ 1, DEV_WAIT_SMEM_EMPTY, abort_flag, status);
          mbar_arrive_expect_tx(&bars->full[s], W_BYTES + L::X_BYTES);
          tma_load_2d_hint(smem + L::OFF_W + s * W_BYTES, &tm_w, &bars->full[s], kb * BK, nb * 128, pol_w);
        }
        tma_load_2d_hint(smem + L::OFF_X + s * L::X_BYTES, &tm_x, &bars->full[s], kb * BK, 0, pol_x);
      }
    }
    if constexpr (CLUSTER) {
      __syncwarp();
      cluster_sync_all();  // every CTA's ring is idle
      cluster_sync_all();  // partial tiles have been delivered to the leader
    }
  }
  else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*e4m3*/ 0, 0, 0, 0, 128, MP);
      uint32_t           it    = 0;
      for (uint32_t u = u_begin; u < u_end; ++u, ++it) {
        const uint32_t s  = it % L::STAGES;
        const uint32_t ph = (it / L::STAGES) & 1;
        const uint32_t p  = s;
        const uint32_t pp = ph;
        mbar_wait(&bars->part_empty[p], pp ^ 1, DEV_WAIT_TMEM_EMPTY, abort_flag, status);
        mbar_wait(&bars->full[s], ph, DEV_WAIT_SMEM_FULL, abort_flag, status);
        if (it == 0) {
          PROFD(2);
        }
        tc_fence_after_sync();
        const uint64_t dw = make_smem_desc_sw128(smem_u32(smem + L::OFF_W + s * W_BYTES), 0, 1024);
        const uint64_t dx = make_smem_desc_sw128(smem_u32(smem + L::OFF_X + s * L::X_BYTES), 0, 1024);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          tc_mma_f8(tmem_base + p * L::PART_COLS, dw + (uint64_t)((kk * UMMA_K) >> 4), dx + (uint64_t)((kk * UMMA_K) >> 4), idesc, kk != 0);
        }
        tc_commit(&bars->part_full[p]);
      }
      PROFD(3);
    }
    if constexpr (CLUSTER) {
      __syncwarp();
      cluster_sync_all();
      cluster_sync_all();
    }
  }
  else {
    // ------------------------------------------- promotion + epilogue ----
    const int      quarter = warp & 3;
    const int      ew      = warp - 2;             // 0..3, index into bars->amax
    const int      n_local = quarter * 32 + lane;  // output column inside the group == TMEM lane
    const int      et      = threadIdx.x - 64;     // 0..127
    const uint32_t t_lane  = (uint32_t)(quarter * 32) << 16;
    uint32_t       it      = 0;

    uint32_t u     = u_begin;
    bool     first = true;  // a cluster CTA runs its one segment even if it is empty: it owes two cluster barriers
    while (u < u_end || (CLUSTER && first)) {
      first = false;
      const int      nb   = (int)(u / (uint32_t)KB);
      const int      kb0  = (int)(u % (uint32_t)KB);
      const uint32_t left = u_end - u;
      const int      kb1  = (left < (uint32_t)(KB - kb0)) ? kb0 + (int)left : KB;
      const bool     whole = (kb0 == 0 && kb1 == KB);

      float acc[MP];
#pragma unroll
      for (int i = 0; i < MP; ++i) {
        acc[i] = 0.0f;
      }
      // Scale operands: lane l of every warp holds A_s[kb, l] and A_s[kb, 32 + l] (fetched one K-block
      // ahead) times B_s; column m's product is broadcast with a shuffle where it is used.
      float a_lo = (lane < M) ? __ldg(A_s + (size_t)kb0 * M + lane) : 0.0f;
      float a_hi = (MP > 32 && lane + 32 < M) ? __ldg(A_s + (size_t)kb0 * M + 32 + lane) : 0.0f;
      float b_nx = __ldg(B_s + (size_t)nb * KB + kb0);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const uint32_t p  = it % L::STAGES;
        const uint32_t pp = (it / L::STAGES) & 1;
        // one fp32 rounding of each scale product, as in the reference
        const float sc_lo = __fmul_rn(a_lo, b_nx);
        const float sc_hi = __fmul_rn(a_hi, b_nx);
        if (kb + 1 < kb1) {
          a_lo = (lane < M) ? __ldg(A_s + (size_t)(kb + 1) * M + lane) : 0.0f;
          a_hi = (MP > 32 && lane + 32 < M) ? __ldg(A_s + (size_t)(kb + 1) * M + 32 + lane) : 0.0f;
          b_nx = __ldg(B_s + (size_t)nb * KB + kb + 1);
        }
        mbar_wait(&bars->part_full[p], pp, DEV_WAIT_TMEM_FULL, abort_flag, status);
        tc_fence_after_sync();
        uint32_t v[MP];
#pragma unroll
        for (int c = 0; c < MP / 16; ++c) {
          tmem_ld_32x32b_x16(tmem_base + p * L::PART_COLS + t_lane + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&v[c * 16]));
        }
        tmem_ld_wait();
        // the partial is in registers: hand the stage back before any arithmetic
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->part_empty[p]);
        }
#pragma unroll
        for (int m = 0; m < MP; ++m) {
          const float sc = __shfl_sync(0xffffffffu, (m < 32) ? sc_lo : sc_hi, m & 31);
          acc[m]         = __fmaf_rn(__uint_as_float(v[m]), sc, acc[m]);
        }
      }
      u += (uint32_t)(kb1 - kb0);
      if (et == 0) {
        PROFD(4);
#ifdef LLMMM_PROFILE
        g_prof_cta[blockIdx.x][1] = global_timer_ns();
#endif
      }

      bool finish = whole;
      if constexpr (CLUSTER) {
        float* red = reinterpret_cast<float*>(smem + L::OFF_W);  // the leader's idle ring: [rank-1][row][n]
        cluster_sync_all();                                      // all MMAs of all CTAs are done: rings idle
        if (c_rank != 0) {
          const uint32_t base = mapa_shared(smem_u32(red + ((size_t)(c_rank - 1) * MP) * 128 + n_local), 0);
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            if (i < M) {
              asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(base + (uint32_t)i * 512u), "f"(acc[i]) : "memory");
            }
          }
        }
        cluster_sync_all();  // release/acquire at cluster scope: the stores above are visible to the leader
        finish = (c_rank == 0);
        if (finish) {
          for (uint32_t rr = 1; rr < c_size; ++rr) {  // fixed order: the result does not depend on timing
#pragma unroll
            for (int i = 0; i < MP; ++i) {
              if (i < M) {
                acc[i] += red[((size_t)(rr - 1) * MP + i) * 128 + n_local];
              }
            }
          }
        }
      }
      else if (!whole) {
        // publish this CTA's partial, then see whether it was the last to arrive
        const int slot = blockIdx.x * 2 + (kb0 == 0 ? 1 : 0);  // run begins inside the group -> slot 0
        float*    dst  = partials + (size_t)slot * (MP * 128);
#pragma unroll
        for (int i = 0; i < MP; ++i) {
          if (i < M) {
            __stcg(dst + i * 128 + n_local, acc[i]);
          }
        }
        __threadfence();
        epilogue_bar_sync();
        if (et == 0) {
          PROFD(5);
        }
        PROFF(0);
        const int c_lo = cta_of_unit((uint32_t)nb * (uint32_t)KB, G, U);
        const int c_hi = cta_of_unit((uint32_t)(nb + 1) * (uint32_t)KB - 1, G, U);
        if (et == 0) {
          const uint32_t old = atomicAdd(&counters[nb], 1u);
          const bool     lst = (old == (uint32_t)(c_hi - c_lo));
          if (lst) {
            counters[nb] = 0;  // ready for the next launch
          }
          bars->last_flag = lst ? 1u : 0u;
        }
        epilogue_bar_sync();
        if (et == 0) {
          PROFD(6);
        }
        PROFF(1);
        finish = bars->last_flag != 0;
        if (finish) {
          __threadfence();
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            acc[i] = 0.0f;
          }
          // Contributors are added in ascending CTA order (the result does not depend on who arrived
          // last); four contributors' loads are in flight together, since each is an L2 round trip.
          for (int c0 = c_lo; c0 <= c_hi; c0 += 4) {
            const float* src[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int c = (c0 + j <= c_hi) ? c0 + j : c_hi;
              // CTA c's run begins inside this group (slot 0) unless it began earlier (slot 1)
              const uint32_t cs = ((uint32_t)c * U) / G;
              const int      sl = c * 2 + ((int)(cs / (uint32_t)KB) == nb && (cs % (uint32_t)KB) != 0 ? 0 : 1);
              src[j]             = partials + (size_t)sl * (MP * 128) + n_local;
            }
#pragma unroll
            for (int i0 = 0; i0 < MP; i0 += 16) {
              if (i0 < M) {
                float t[4][16];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                  for (int i = 0; i < 16; ++i) {
                    t[j][i] = (i0 + i < M) ? __ldcg(src[j] + (i0 + i) * 128) : 0.0f;
                  }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (c0 + j <= c_hi) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                      acc[i0 + i] += t[j][i];
                    }
                  }
                }
              }
            }
          }
        }
        epilogue_bar_sync();  // last_flag may be rewritten by the next segment
        PROFF(2);
      }

      if (finish) {
        const size_t n_glob = (size_t)nb * 128 + n_local;
        if constexpr (OUT_F32) {
          float* C = reinterpret_cast<float*>(C_out);
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            if (i < M) {
              C[(size_t)i * N + n_glob] = acc[i];
            }
          }
        }
        else {
          // group absmax over the 128 lanes: one warp-wide integer max per row (the bit pattern of a
          // non-negative float orders like the float), then 4 warps through shared memory
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            if (i < M) {
              const uint32_t a = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(acc[i])));
              if (lane == 0) {
                bars->amax[ew][i] = __uint_as_float(a);
              }
            }
          }
          epilogue_bar_sync();
          PROFF(3);
          // thread i finishes row i's absmax and does the two divisions once for everybody
          if (et < M) {
            const float amax = fmaxf(fmaxf(bars->amax[0][et], bars->amax[1][et]), fmaxf(bars->amax[2][et], bars->amax[3][et]));
            bars->inv[et]    = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
            C_s[(size_t)nb * M + et] = __fdiv_rn(amax, 448.0f);
          }
          epilogue_bar_sync();
          uint8_t* C = reinterpret_cast<uint8_t*>(C_out);
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            if (i < M) {
              C[(size_t)i * N + n_glob] = (uint8_t)__nv_cvt_float_to_fp8(acc[i] * bars->inv[i], __NV_SATFINITE, __NV_E4M3);
            }
          }
          epilogue_bar_sync();  // bars->amax and bars->inv are reused by the next segment
          PROFF(4);
        }
      }
    }
#ifdef LLMMM_PROFILE
    if (et == 0) {
      g_prof_cta[blockIdx.x][2] = global_timer_ns();
    }
#endif
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    PROFD(7);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
  if (threadIdx.x == 32) {
    PROFD(8);
#ifdef LLMMM_PROFILE
    g_prof_cta[blockIdx.x][3] = global_timer_ns();
#endif
  }
}

#ifdef LLMMM_PROFILE
extern "C" void llmmm_profile_dump_pdl()
{
  unsigned long long c[256][4], w[256][2];
  cudaMemcpyFromSymbol(c, g_prof_cta, sizeof(c));
  cudaMemcpyFromSymbol(w, g_prof_pdl, sizeof(w));
  double held = 0, setup = 0; unsigned long long first_entry = ~0ull, last_entry = 0, last_exit = 0, first_go = ~0ull; int n = 0;
  for (int i = 0; i < 256; ++i) {
    if (c[i][0] == 0 || w[i][1] == 0) continue;
    held += (double)(w[i][1] - w[i][0]); setup += (double)(w[i][0] - c[i][0]); ++n;
    if (c[i][0] < first_entry) first_entry = c[i][0];
    if (c[i][0] > last_entry) last_entry = c[i][0];
    if (c[i][3] > last_exit) last_exit = c[i][3];
    if (w[i][1] < first_go) first_go = w[i][1];
  }
  unsigned long long st[256][4];
  cudaMemcpyFromSymbol(st, g_prof_set, sizeof(st));
  printf("CTA 5: entry +0, barriers initialised +%llu, tcgen05.alloc from +%llu to +%llu, CTA barrier passed +%llu, at the dependency wait +%llu, released +%llu, exit +%llu ns\n",
         st[5][0] - c[5][0], st[5][1] - c[5][0], st[5][2] - c[5][0], st[5][3] - c[5][0], w[5][0] - c[5][0], w[5][1] - c[5][0], c[5][3] - c[5][0]);
  unsigned long long h[16];
  cudaMemcpyFromSymbol(h, g_prof_dec, sizeof(h));
  printf("CTA 0 after its release (ns): first operands +%lld, MMAs issued +%lld, promotion done +%lld, all roles done +%lld, TMEM freed +%lld\n",
         (long long)(h[2] - w[0][1]), (long long)(h[3] - w[0][1]), (long long)(h[4] - w[0][1]), (long long)(h[7] - w[0][1]), (long long)(h[8] - w[0][1]));
  printf("last launch, %d CTAs: entries spread over %llu ns, set-up %.0f ns, held at the dependency wait %.0f ns (avg), "
         "first entry -> first release %llu ns, first entry -> last exit %llu ns\n", n, last_entry - first_entry, setup / n,
         held / n, first_go - first_entry, last_exit - first_entry);
}

extern "C" void llmmm_profile_dump_decode()
{
  unsigned long long h[16];
  unsigned long long c[256][4];
  cudaMemcpyFromSymbol(c, g_prof_cta, sizeof(c));
  unsigned long long t0 = ~0ull, t_last_entry = 0, t_loop = 0, t_exit = 0;
  for (int i = 0; i < 148; ++i) {
    if (c[i][0] == 0) continue;
    if (c[i][0] < t0) t0 = c[i][0];
    if (c[i][0] > t_last_entry) t_last_entry = c[i][0];
    if (c[i][1] > t_loop) t_loop = c[i][1];
    if (c[i][3] > t_exit) t_exit = c[i][3];
  }
  printf("all CTAs (ns from first entry): last entry %llu, last promotion loop done %llu, last exit %llu\n",
         t_last_entry - t0, t_loop - t0, t_exit - t0);
  unsigned long long f[256][6];
  cudaMemcpyFromSymbol(f, g_prof_fin, sizeof(f));
  int worst = 0;
  for (int i = 0; i < 148; ++i) {
    if (c[i][3] > c[worst][3]) worst = i;
  }
  printf("slowest CTA %d (ns from first entry): entry %llu loop done %llu | published %llu counted %llu reduced %llu amax %llu stored %llu | "
         "roles done %llu exit %llu\n",
         worst, c[worst][0] - t0, c[worst][1] - t0, f[worst][0] - t0, f[worst][1] - t0, f[worst][2] - t0, f[worst][3] - t0,
         f[worst][4] - t0, c[worst][2] - t0, c[worst][3] - t0);
  cudaMemcpyFromSymbol(h, g_prof_dec, sizeof(h));
  printf("decode CTA 0 (ns from kernel entry): set-up done %llu, first operands %llu, MMAs issued %llu, promotion done %llu, "
         "partial published %llu, arrival counted %llu, all roles done %llu, TMEM freed %llu\n",
         h[1] - h[0], h[2] - h[0], h[3] - h[0], h[4] - h[0], h[5] - h[0], h[6] - h[0], h[7] - h[0], h[8] - h[0]);
}
#endif

// ------------------------------------------------------------ host side ---

std::atomic<int> g_static_weights{0};  // llmmm_set_static_weights()

namespace {
static_assert(deccfg::COUNTER_BYTES == WS_DECODE_COUNTER_BYTES, "layout of the registered scratch");
Workspace  g_ws[64];
std::mutex g_ws_mutex;

int padded_m(int M)
{
  return M <= 16 ? 16 : (M <= 32 ? 32 : 64);
}
}  // namespace

size_t decode_workspace_bytes(int M)
{
  return WS_HEADER_BYTES + (size_t)deccfg::MAX_CTAS * 2 * padded_m(M) * 128 * sizeof(float);
}

Workspace registered_workspace(int device)
{
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  return g_ws[device];
}

template<int MP, bool OUT_F32>
static int launch_decode_t(const void*       A,
                           const float*      A_s,
                           const void*       B,
                           const float*      B_s,
                           void*             C,
                           float*            C_s,
                           int               M,
                           int               N,
                           int               K,
                           uint32_t*         counters,
                           float*            partials,
                           const DeviceInfo* info,
                           cudaStream_t      stream)
{
  using namespace deccfg;
  using L = DecodeSmem<MP>;
  CUtensorMap tm_w, tm_x;
  if (!make_tmap_2d(&tm_w, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_x, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, MP, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(cudaFuncSetAttribute(
      fp8_decode_kernel<MP, OUT_F32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM_BYTES));
    attr_set[info->device] = true;
  }
  const long long U = (long long)(N / 128) * (K / BK);
  int             G = info->sm_count < MAX_CTAS ? info->sm_count : MAX_CTAS;
  if ((long long)G > U) {
    G = (int)U;
  }
  LLMMM_CUDA_TRY(launch_pdl(fp8_decode_kernel<MP, OUT_F32, false>, dim3((unsigned)G), dim3(THREADS), L::SMEM_BYTES, stream,
                            1, tm_w, tm_x, A_s, B_s, C, C_s, M, N, K, partials, counters, g_static_weights.load(),
                            info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

template<int MP, bool OUT_F32>
static int launch_decode_cluster_t(const void*       A,
                                   const float*      A_s,
                                   const void*       B,
                                   const float*      B_s,
                                   void*             C,
                                   float*            C_s,
                                   int               M,
                                   int               N,
                                   int               K,
                                   int               cluster,
                                   const DeviceInfo* info,
                                   cudaStream_t      stream)
{
  using namespace deccfg;
  using L = DecodeSmem<MP>;
  CUtensorMap tm_w, tm_x;
  if (!make_tmap_2d(&tm_w, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
      || !make_tmap_2d(&tm_x, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, MP, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LLMMM_ERR_CUDA;
  }
  static thread_local bool attr_set[64] = {};
  if (!attr_set[info->device]) {
    LLMMM_CUDA_TRY(cudaFuncSetAttribute(
      fp8_decode_kernel<MP, OUT_F32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM_BYTES));
    attr_set[info->device] = true;
  }
  float*    no_partials = nullptr;
  uint32_t* no_counters = nullptr;
  LLMMM_CUDA_TRY(launch_pdl(fp8_decode_kernel<MP, OUT_F32, true>, dim3((unsigned)((N / 128) * cluster)), dim3(THREADS),
                            L::SMEM_BYTES, stream, (unsigned)cluster, tm_w, tm_x, A_s, B_s, C, C_s, M, N, K, no_partials,
                            no_counters, g_static_weights.load(), info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

namespace {
// How many clusters of `size` CTAs (one CTA per SM, as the decode kernel needs) the device can hold at once.
int cluster_capacity(const DeviceInfo* info, int size)
{
  static std::mutex mu;
  static int        cache[64][9];
  static bool       known[64][9];
  std::lock_guard<std::mutex> lock(mu);
  if (!known[info->device][size]) {
    using L = DecodeSmem<64>;
    int clusters = 0;
    if (cudaFuncSetAttribute(fp8_decode_kernel<64, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM_BYTES)
        == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim            = dim3((unsigned)(size * (info->sm_count / size)));
      cfg.blockDim           = dim3(deccfg::THREADS);
      cfg.dynamicSmemBytes   = L::SMEM_BYTES;
      cudaLaunchAttribute attr[1];
      attr[0].id               = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = (unsigned)size;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs                = attr;
      cfg.numAttrs             = 1;
      if (cudaOccupancyMaxActiveClusters(&clusters, fp8_decode_kernel<64, false, true>, &cfg) != cudaSuccess) {
        clusters = 0;
      }
    }
    cudaGetLastError();
    cache[info->device][size] = clusters;
    known[info->device][size] = true;
  }
  return cache[info->device][size];
}

// Largest allowed cluster size for which every output group gets a resident cluster and every CTA at least
// one K-block; 0 when the cluster path does not apply (then stream-K with scratch is used).
int choose_cluster(const DeviceInfo* info, int M, int N, int K)
{
  const int groups = N / 128, kb = K / 128;
  // Remote shared-memory stores are slow (measured: two peers delivering 32 KB each take about 4 us), so the
  // cluster path is used only while the partial tiles are small: not for M > 32, at most 4 CTAs for M > 16.
  if (M > 32) {
    return 0;
  }
  const int max_size = (M > 16) ? 4 : 7;
  for (int size = max_size; size >= 2; --size) {
    if (kb >= size && groups * size <= info->sm_count && cluster_capacity(info, size) >= groups) {
      // worth it only if the clusters occupy at least half of the SMs; otherwise stream-K spreads the weight
      // blocks over all of them
      return (groups * size * 2 >= info->sm_count) ? size : 0;
    }
  }
  return 0;
}
}  // namespace

bool describe_decode_plan(const DeviceInfo* info, int M, int N, int K, char* buf, size_t len)
{
  if (M > 64 || N / 128 > deccfg::MAX_GROUPS || (long long)(N / 128) * (K / 128) * 256 >= (1ll << 31)) {
    return false;
  }
  const int mp = padded_m(M);
  if (const int cluster = choose_cluster(info, M, N, K)) {
    snprintf(buf, len, "fp8_decode_kernel<%d, cluster>: %d output groups x clusters of %d CTAs, each CTA streams %d or %d of the "
             "%d K-blocks; reduction through distributed shared memory, no scratch", mp, N / 128, cluster, (K / 128) / cluster,
             (K / 128 + cluster - 1) / cluster, K / 128);
    return true;
  }
  const Workspace ws = registered_workspace(info->device);
  if (ws.ptr == nullptr || ws.bytes < decode_workspace_bytes(M)) {
    return false;  // no scratch: the general kernel runs
  }
  const long long U = (long long)(N / 128) * (K / 128);
  long long       G = info->sm_count < deccfg::MAX_CTAS ? info->sm_count : deccfg::MAX_CTAS;
  G                 = G < U ? G : U;
  snprintf(buf, len, "fp8_decode_kernel<%d, stream-K>: %lld weight blocks of 128x128 over %lld CTAs (%.1f each), partial tiles "
           "through the registered scratch, last-arriving CTA reduces", mp, U, G, (double)U / (double)G);
  return true;
}

int warm_decode_kernels(const DeviceInfo* info)
{
#define LLMMM_WARM_DECODE(MPV, F32, CL)                                                                                \
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_decode_kernel<MPV, F32, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                      (int)DecodeSmem<MPV>::SMEM_BYTES));
  LLMMM_WARM_DECODE(16, false, false) LLMMM_WARM_DECODE(16, true, false) LLMMM_WARM_DECODE(16, false, true) LLMMM_WARM_DECODE(16, true, true)
  LLMMM_WARM_DECODE(32, false, false) LLMMM_WARM_DECODE(32, true, false) LLMMM_WARM_DECODE(32, false, true) LLMMM_WARM_DECODE(32, true, true)
  LLMMM_WARM_DECODE(64, false, false) LLMMM_WARM_DECODE(64, true, false) LLMMM_WARM_DECODE(64, false, true) LLMMM_WARM_DECODE(64, true, true)
#undef LLMMM_WARM_DECODE
  for (int size = 2; size <= 7; ++size) {
    cluster_capacity(info, size);  // occupancy queries, cached
  }
  return LLMMM_OK;
}

// Returns -1 when the decode path does not apply (M > 64, too many groups, or
// no scratch buffer large enough is registered): the caller then uses the
// general kernel, which needs no scratch.
int launch_decode(bool         out_f32,
                  const void*  A,
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
  if (M > 64 || N / 128 > deccfg::MAX_GROUPS || (long long)(N / 128) * (K / 128) * 256 >= (1ll << 31)) {
    return -1;
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  const int mp = padded_m(M);
  if (const int cluster = choose_cluster(info, M, N, K)) {
#define LLMMM_DECODE_CLUSTER_CASE(MPV)                                                                                 \
  if (mp == MPV) {                                                                                                     \
    return out_f32 ? launch_decode_cluster_t<MPV, true>(A, A_s, B, B_s, C, C_s, M, N, K, cluster, info, stream) :      \
                     launch_decode_cluster_t<MPV, false>(A, A_s, B, B_s, C, C_s, M, N, K, cluster, info, stream);      \
  }
    LLMMM_DECODE_CLUSTER_CASE(16)
    LLMMM_DECODE_CLUSTER_CASE(32)
    LLMMM_DECODE_CLUSTER_CASE(64)
#undef LLMMM_DECODE_CLUSTER_CASE
  }
  const Workspace ws = registered_workspace(info->device);
  if (ws.ptr == nullptr || ws.bytes < decode_workspace_bytes(M)) {
    return -1;
  }
  uint32_t* counters = static_cast<uint32_t*>(ws.ptr);
  float*    partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws.ptr) + WS_HEADER_BYTES);
#define LLMMM_DECODE_CASE(MPV)                                                                                         \
  if (mp == MPV) {                                                                                                     \
    return out_f32 ? launch_decode_t<MPV, true>(A, A_s, B, B_s, C, C_s, M, N, K, counters, partials, info, stream) :   \
                     launch_decode_t<MPV, false>(A, A_s, B, B_s, C, C_s, M, N, K, counters, partials, info, stream);   \
  }
  LLMMM_DECODE_CASE(16)
  LLMMM_DECODE_CASE(32)
  LLMMM_DECODE_CASE(64)
#undef LLMMM_DECODE_CASE
  return -1;
}

}  // namespace llmmm

extern "C" {

size_t llmmm_fp8_workspace_bytes(int M, int N, int K)
{
  (void)K;
  if (M < 1 || N < 128) {
    return 0;
  }
  if (M > 64) {
    return llmmm::split_workspace_bytes();  // the pair kernel's split tiles (65..128 rows use it for few-tile shapes)
  }
  if (N / 128 > llmmm::deccfg::MAX_GROUPS) {
    return 0;
  }
  return llmmm::decode_workspace_bytes(M);
}

int llmmm_set_static_weights(int enabled)
{
  llmmm::g_static_weights.store(enabled ? 1 : 0);
  return LLMMM_OK;
}

int llmmm_set_workspace(void* device_ptr, size_t bytes)
{
  using namespace llmmm;
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  if (device_ptr != nullptr) {
    if (((uintptr_t)device_ptr & 255) != 0 || bytes < WS_HEADER_BYTES) {
      return set_error(LLMMM_ERR_SHAPE, "workspace must be 256-byte aligned and at least %zu bytes", WS_HEADER_BYTES);
    }
    // the arrival counters must start at zero; every launch leaves them at zero again
    LLMMM_CUDA_TRY(cudaMemset(device_ptr, 0, WS_HEADER_BYTES));
  }
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  g_ws[info->device].ptr   = device_ptr;
  g_ws[info->device].bytes = device_ptr ? bytes : 0;
  return LLMMM_OK;
}

}  // extern "C"

// ------------------------------------------------ entry point without scratch --
//
// Some callers have no way to hand this library a scratch buffer: a serving
// process that gave every byte of device memory to its own pool at start-up
// (a later cudaMalloc fails there, or fragments the pool), or a decode loop
// that must not meet cudaMalloc / cudaFree at all because those calls
// synchronise the whole device and stall every other stream.  For them the
// split-K scratch of the decode kernel lives in the library image itself: one
// fixed array per GPU that loads the library, sized for the smallest
// activation tile (M <= 16).  Nothing is allocated on any call.
namespace llmmm {
namespace {

constexpr int    NOALLOC_MAX_M = 16;
constexpr size_t NOALLOC_BYTES = deccfg::COUNTER_BYTES + (size_t)deccfg::MAX_CTAS * 2 * 16 * 128 * sizeof(float);

// 16 KB of arrival counters followed by 256 x 2 partial tiles of 16 x 128 fp32: 4,210,688 bytes.
static __device__ __align__(256) uint8_t g_noalloc_scratch[NOALLOC_BYTES];

// In host code the array's name is only a handle for the runtime; the device
// address is looked up once per device (with that device current) and kept.
uint8_t*   g_noalloc_ptr[64];
bool       g_noalloc_ready[64];
std::mutex g_noalloc_mutex;

int noalloc_scratch(const DeviceInfo* info, uint8_t** out)
{
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ready[info->device]) {
    uint8_t*    ptr = nullptr;
    cudaError_t e   = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      return set_error(LLMMM_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
    }
    g_noalloc_ptr[info->device]   = ptr;
    g_noalloc_ready[info->device] = true;
  }
  *out = g_noalloc_ptr[info->device];
  return LLMMM_OK;
}

}  // namespace
}  // namespace llmmm

extern "C" int llmmm_fp8_blockwise_mm_e4m3out_noalloc(const void*    A,
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
  using namespace llmmm;
  if (A == nullptr || A_scale_t == nullptr || B_t == nullptr || B_scale_t == nullptr || C == nullptr
      || C_scale_t == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (N < 128 || K < 128 || (N % 128) != 0 || (K % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "N or K are not aligned. (need N%%128==0, K%%128==0; got %d %d)", N, K);
  }
  if (M < 1 || M > NOALLOC_MAX_M || N / 128 > deccfg::MAX_GROUPS
      || (long long)(N / 128) * (K / 128) * 256 >= (1ll << 31)) {
    return set_error(LLMMM_ERR_SHAPE,
                     "the entry point without scratch takes 1 <= M <= %d and N <= %d (its built-in scratch is %zu bytes); "
                     "got M=%d N=%d: use llmmm_fp8_blockwise_mm_e4m3out with a caller-owned workspace",
                     NOALLOC_MAX_M,
                     deccfg::MAX_GROUPS * 128,
                     NOALLOC_BYTES,
                     M,
                     N);
  }
  if (((uintptr_t)A | (uintptr_t)B_t | (uintptr_t)C) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "A, B and C must be 16-byte aligned");
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  uint8_t* scratch = nullptr;
  int      rc      = noalloc_scratch(info, &scratch);
  if (rc != LLMMM_OK) {
    return rc;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (const int cluster = choose_cluster(info, M, N, K)) {
    // same choice as llmmm_fp8_blockwise_mm_e4m3out makes: the cluster kernel needs no scratch at all
    return launch_decode_cluster_t<16, false>(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K, cluster, info, s);
  }
  // The array keeps whatever the previous call left.  Partial tiles are always
  // written before they are read, but the arrival counters of the groups this
  // call uses must start at zero.
  LLMMM_CUDA_TRY(cudaMemsetAsync(scratch, 0, (size_t)(N / 128) * sizeof(uint32_t), s));
  return launch_decode_t<16, false>(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K,
                                    reinterpret_cast<uint32_t*>(scratch),
                                    reinterpret_cast<float*>(scratch + deccfg::COUNTER_BYTES), info, s);
}

