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
//   * stream-K: all SMs stream the same number of weight blocks whatever N is:
//     the (N/128 x K/128) grid of weight blocks is cut into contiguous runs, one
//     or two per CTA; a run crosses output groups, giving "segments".  With at
//     least as many groups as CTAs every CTA takes floor(groups / CTAs) whole
//     groups, and only the left-over groups are cut evenly among the CTAs,
//     which work on those cut pieces FIRST;
//   * warp 0 streams weight blocks (and the matching activation slab) through
//     a 6-8-deep TMA ring; warps 1-3 take turns issuing the MMAs of a K-block
//     (four per K-block, from zero, into the tensor-memory partial stage of the
//     ring slot): a thread that issues four MMAs and a commit is held for about
//     640 clk whatever their width, so one thread alone could not keep up with
//     the ring; the promotion warps (4, or 8 for 32 and 64 columns) promote
//     with acc = fma(partial, A_s*B_s, acc) in registers, the scale products of
//     a whole run staged through shared memory ahead of time (a load per
//     K-block would put an L2 round trip into every iteration);
//   * a segment that covers a group's whole K range is finished in place;
//     otherwise its fp32 partial goes to the caller's scratch buffer as
//     self-announcing words (zero = not there yet), and the rows of the output
//     group are shared out among the contributors' REDUCTION warps, a fourth
//     warpgroup of the stream-K kernel that works beside the promotion warps (a
//     reduce-scatter: one warp reads one row's words of every contributor, adds
//     them in fixed CTA order, takes the absmax, quantises and stores the row),
//     so results do not depend on timing, no single CTA reads every partial
//     tile, the exchange costs one store and one load latency instead of store
//     + fence + atomic + poll + load, and when whole groups follow the cut
//     pieces that latency passes while the CTA is still streaming;
//   * the 1x128 output group runs across the 128 lanes in this orientation:
//     for a whole segment the group absmax is a warp-shuffle reduction plus a
//     4-entry exchange in shared memory between the four warps.
#include <array>
#include <cuda_fp8.h>
#include <map>
#include <mutex>
#include <vector>

#include "host_common.h"
#include "sm100.cuh"

namespace llmmm {

namespace deccfg {
constexpr int      BK            = 128;
constexpr int      UMMA_K        = 32;
constexpr int      MAX_STAGES    = 8;    // the ring depth depends on the activation tile, see DecodeSmem
// warps 0-3: producer, three MMA issuers; warps 4-7 (up to 16 activation columns) or 4-11 (32, 64 columns): promotion.
// With 64 columns one promotion warp per scheduler could not keep up with the weight stream (measured: ~600 ns per
// K-block, all of it latency: shared-memory loads, the barrier, tensor-memory loads, 64 FMAs, one after the other
// with nothing to overlap; HBM delivers a block every 364 ns): two warps per scheduler take half of the columns
// each (M = 64: 9.8 / 8.2 / 22.2 / 12.0 -> 7.6 / 6.9 / 17.0 / 9.6 us on the four Qwen3-4B shapes; M = 32, together
// with an SM to itself and eight stages: 7.8 / 6.5 / 17.1 / 9.5 -> 6.6 / 5.5 / 14.7 / 8.0 us).
constexpr int      EPI_WARP0     = 4;    // first promotion warp (setmaxnreg acts on whole warpgroups of 4 warps)
constexpr int      REGS_CTRL     = 56;   // the control warpgroup gives up registers ...
constexpr int      REGS_EPI      = 200;  // ... and the promotion and reduction warpgroups take them
__host__ __device__ constexpr int promo_warps(int mp) { return mp > 16 ? 8 : 4; }
// The stream-K kernel has one more warpgroup: it adds up the partial tiles of the output groups that were cut
// among CTAs while the promotion warps are still streaming (see the kernel).  The cluster kernel has none.
__host__ __device__ constexpr int reduce_warps(bool cluster) { return cluster ? 0 : 4; }
__host__ __device__ constexpr int threads(int mp, bool cluster) { return 128 + 32 * (promo_warps(mp) + reduce_warps(cluster)); }
// Up to 16 activation columns a CTA takes half an SM (shared memory, tensor memory, registers), so that the
// kernels before and after it in a launch chain are resident beside it: set up, waiting for their turn, or
// finishing.  (Measured on a Qwen3-4B MLP block of four launches at M = 1: 22.7 us; with the stream-K kernel on a
// whole SM 25.8 us, although that kernel alone is faster that way, 11.1 against 12.1 us.)
__host__ __device__ constexpr int ctas_per_sm(int mp, bool cluster) { return mp <= 16 ? 2 : 1; }
// Registers per thread after setmaxnreg, by kernel form.  What a thread starts with (ptxas reports it): 128 with
// 256 threads and two CTAs per SM, 80 with 384 threads and two CTAs, 168 with 384 threads and one, 128 with 512;
// setmaxnreg moves registers inside the CTA's allocation and waits for ever if it asks for more.
//   cluster kernel                 : control 56, promotion 200
//   stream-K, 16 columns (2 / SM)  : control 56, promotion 88, reduction 96   (384 x 80 = 30720)
//   stream-K, 32 / 64 columns      : control 56, promotion 128 (as launched), reduction 200   (512 x 128 = 65536)
__host__ __device__ constexpr int regs_promo(int mp, bool cluster) { return cluster ? REGS_EPI : (mp <= 16 ? 88 : 128); }
__host__ __device__ constexpr int regs_reduce(int mp) { return mp <= 16 ? 96 : REGS_EPI; }
static_assert(128 * REGS_CTRL + 128 * regs_promo(16, true) <= 256 * 128, "cluster kernel, 16 columns");
static_assert(128 * REGS_CTRL + 256 * regs_promo(64, true) <= 384 * 168, "cluster kernel, 32 / 64 columns");
static_assert(128 * REGS_CTRL + 128 * regs_promo(16, false) + 128 * regs_reduce(16) <= 384 * 80, "stream-K kernel, 16 columns");
static_assert(128 * REGS_CTRL + 256 * regs_promo(64, false) + 128 * regs_reduce(64) <= 512 * 128, "stream-K kernel, 32 / 64 columns");
constexpr uint32_t W_BYTES       = 128 * BK;
constexpr int      MAX_CTAS      = 160;  // grid of the stream-K kernel: one CTA per SM, at most this many
constexpr int      MAX_GROUPS    = 4096; // N <= 524288
}  // namespace deccfg

template<int MP>
struct DecodeSmem {
  static constexpr uint32_t X_BYTES    = MP * deccfg::BK;
  // Up to 16 activation columns: as deep a ring as lets two CTAs share an SM (113 KB each; tensor memory: 256
  // columns each): the next kernel of a launch chain then sets up, and requests static weights, beside the
  // running one.  With 32 or 64 columns a stage is 20 or 24 KB; measured, an SM to itself and eight stages is
  // faster there (cluster shapes 9.9 / 8.2 / 12.1 us against 11.8 / 9.3 / 14.2 us at M = 64).
  static constexpr int      STAGES     = MP <= 16 ? 6 : 8;
  // K-block `it` uses ring stage it % STAGES and the tensor-memory partial stage of the same index, so ONE
  // tcgen05.commit per K-block tells both the promotion warps (partial ready) and the producer (operands
  // consumed); a second commit would cost the single issuing thread another ~150 clk per K-block.
  static constexpr uint32_t PART_COLS  = MP < 32 ? 32 : MP;
  static constexpr uint32_t TMEM_COLS  = STAGES * PART_COLS <= 256 ? 256 : 512;  // one partial stage per ring stage
  static_assert(STAGES * PART_COLS <= TMEM_COLS, "partial stages exceed the tensor memory allocation");
  static constexpr uint32_t OFF_W      = 0;
  static constexpr uint32_t OFF_X      = STAGES * deccfg::W_BYTES;
  static constexpr uint32_t OFF_BAR    = OFF_X + STAGES * X_BYTES;
  // cluster kernel: the idle ring holds the CTA's own partial tile (MP rows of 512 bytes) and what it receives,
  // c * ceil(M / c) < MP + 8 rows
  static_assert((2 * MP + 8) * 512 <= STAGES * (deccfg::W_BYTES + X_BYTES), "partial tiles must fit into the idle ring");
  // scale products A_s[kb, m] * B_s[nb, kb] of CHUNK consecutive K-blocks of the CTA's run, [CHUNK][MP] fp32
  static constexpr int      CHUNK      = MP <= 32 ? 32 : 16;
  static constexpr uint32_t OFF_SC     = OFF_BAR + 1536;
  static constexpr uint32_t SC_BYTES   = CHUNK * MP * 4;
  // at least 80 KB, so that never more than two CTAs share an SM: a third one would sit in tcgen05.alloc until
  // tensor memory is freed
  static constexpr uint32_t USED_BYTES = OFF_SC + SC_BYTES + 1024;
  static_assert(MP > 16 || 2 * (USED_BYTES + 1024) <= 228 * 1024, "two CTAs of consecutive launches must fit on one SM");
  static_assert(USED_BYTES <= 227 * 1024, "shared memory of one CTA");
  static constexpr uint32_t SMEM_BYTES = USED_BYTES > 80 * 1024 ? USED_BYTES : 80 * 1024;
};

struct DecodeBars {
  uint64_t full[deccfg::MAX_STAGES];        // operands of the stage have landed
  uint64_t part_full[deccfg::MAX_STAGES];   // the K-block's MMAs are done: partial ready, operands consumed
  uint64_t part_empty[deccfg::MAX_STAGES];  // the promotion warps have copied the partial out
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t pad[2];
  uint64_t red;  // cluster kernel: the other CTAs' partials of this CTA's rows have landed (counted in bytes)
  float    amax[4][64];
  float    inv[64];
};
static_assert(sizeof(DecodeBars) <= 1536, "DecodeBars outgrew its slot in shared memory");

#ifdef LLMMM_PROFILE
// Profiling build only: %globaltimer of every CTA at its phases (see llmmm_profile_dump_decode()).
__device__ unsigned long long g_prof_cta[256][16];
__device__ unsigned long long g_prof_kb[8][4];  // CTA 0, first promotion warp, K-blocks 0..7: waiting, partial seen, loaded, done
#define PROF_KB(i)                                                                                                     \
  do {                                                                                                                 \
    if (blockIdx.x == 0 && threadIdx.x == deccfg::EPI_WARP0 * 32 && it < 8) {                                          \
      g_prof_kb[it][i] = global_timer_ns();                                                                            \
    }                                                                                                                  \
  } while (0)
#define PROF_CTA(i)                                                                                                    \
  do {                                                                                                                 \
    if ((threadIdx.x & 31) == 0) {                                                                                     \
      g_prof_cta[blockIdx.x][i] = global_timer_ns();                                                                   \
    }                                                                                                                  \
  } while (0)
#else
#define PROF_CTA(i)
#define PROF_KB(i)
#endif

template<int NTHREADS>  // all promotion warps of the CTA
__device__ __forceinline__ void epilogue_bar_sync()
{
  asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory");
}

// unit u of the (group, K-block) grid belongs to CTA ((u+1)*G - 1) / U, the
// largest c with floor(c*U/G) <= u.
__device__ __forceinline__ int cta_of_unit(uint32_t u, uint32_t G, uint32_t U)
{
  return (int)(((u + 1) * G - 1) / U);
}

// One output group that was cut among several CTAs, as seen by one promotion warp of a contributor.
struct SplitGroup {
  int  nb;     // output group
  int  c_lo;   // first contributing CTA
  int  cnt;    // contributors
  int  gw;     // this warp's index among the promotion warps of the contributors (4 or 8 per CTA)
  bool mine;   // this warp owns at least one row of the group
};

// Partial tiles travel between CTAs as self-announcing 32-bit words: the scratch is all zero between launches,
// a contributor stores its fp32 values in a code that is never zero, and a reader polls the words themselves
// until none of those it needs is zero.  There is no separate "data is ready" signal and therefore no fence, no
// atomic and no second round trip.  A reader puts the words it consumed back to zero.
// Code: the value's bits with the sign flipped, so +0.0 (frequent) becomes 0x80000000; the one value that would
// then be zero, -0.0 (a product that underflowed), takes the code of a NaN that arithmetic never produces.
constexpr uint32_t PARTIAL_MINUS_ZERO = 0xffc00001u;

__device__ __forceinline__ uint32_t encode_partial(float v)
{
  const uint32_t w = __float_as_uint(v) ^ 0x80000000u;
  return w != 0u ? w : PARTIAL_MINUS_ZERO;
}

__device__ __forceinline__ float decode_partial(uint32_t w)
{
  return __uint_as_float(w != PARTIAL_MINUS_ZERO ? w ^ 0x80000000u : 0x80000000u);
}

__device__ __forceinline__ void st_partial(uint32_t* p, float v)
{
  asm volatile("st.relaxed.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(encode_partial(v)) : "memory");
}

__device__ __forceinline__ uint4 ld_partial4(const uint32_t* p)
{
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// One finished row of one 128-column output group, four columns per lane of one warp: fp32 as it is, or the
// row's absmax (the bit pattern of a non-negative float orders like the float: one warp-wide integer max), the
// two divisions of the quantisation rule, four e4m3 bytes per lane and the scale.
template<bool OUT_F32>
__device__ __forceinline__ void store_group_row(float4 s, int m, int nb, void* __restrict__ C_out, float* __restrict__ C_s,
                                                int M, int N, int lane)
{
  if constexpr (OUT_F32) {
    reinterpret_cast<float4*>(reinterpret_cast<float*>(C_out) + (size_t)m * N + (size_t)nb * 128)[lane] = s;
  }
  else {
    const float    mine = fmaxf(fmaxf(fabsf(s.x), fabsf(s.y)), fmaxf(fabsf(s.z), fabsf(s.w)));
    const float    amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mine)));
    const float    inv  = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
    const uint32_t q    = pack_e4m3x4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
    reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(C_out) + (size_t)m * N + (size_t)nb * 128)[lane] = q;
    if (lane == 0) {
      C_s[(size_t)nb * M + m] = __fdiv_rn(amax, 448.0f);
    }
  }
}

// Cheap wait in front of the reduction of a split group: lane j polls ONE word of contributor j's partial tile (in
// the first row this warp owns: nobody else puts that word back to zero), so that a warp that is early does not
// keep re-reading whole rows of every contributor -- hundreds of warps doing that would load the L2 with
// megabytes per polling round.  Only a hint: stores may land in any order, and the reduction still checks
// every word it uses.  Bounded like every wait.
template<int MP>
__device__ __forceinline__ bool wait_contributors(const SplitGroup& g, const uint32_t* partials, int lane,
                                                  volatile uint32_t* abort_flag, uint32_t* status)
{
  for (int base = 0; base < g.cnt; base += 32) {
    const int          j     = base + lane;
    const uint32_t*    word  = partials + ((size_t)((g.c_lo + j) * 2 + (j == 0 ? 1 : 0)) * MP + g.gw) * 128 + 127;
    unsigned long long t0    = 0;
    uint32_t           spins = 0;
    for (;;) {
      uint32_t w = 1u;
      if (j < g.cnt) {
        asm volatile("ld.relaxed.gpu.global.b32 %0, [%1];" : "=r"(w) : "l"(word) : "memory");
      }
      if (__all_sync(0xffffffffu, w != 0u)) {
        break;
      }
      __nanosleep(200);  // the words may be a whole stream away: leave the memory system to the weights
      if ((++spins & 0x7) == 0) {
        if (*abort_flag) {
          return false;
        }
        const unsigned long long now = global_timer_ns();
        if (t0 == 0) {
          t0 = now;
        }
        else if (now - t0 > WAIT_LIMIT_NS) {
          *abort_flag = DEV_WAIT_SPLITK;
          atomicCAS(status, 0u, (uint32_t)DEV_WAIT_SPLITK);
          return false;
        }
      }
    }
  }
  return true;
}

// Reduce-scatter step of one warp over NG (one or two) split groups at once.  Warp gw of a group's PW * cnt warps
// (PW promotion warps per contributor) owns rows gw, gw + PW cnt, ...; per pass it takes RB of its rows in each group and adds their partial tiles CB
// contributors at a time, ascending CTA order, four columns per lane (a warp reads one 512-byte row per load
// instruction): NG * RB * CB loads are in flight together, so a pass costs one L2 round trip whatever the row
// count, repeated (bounded) while a contributor's words have not landed yet.  Then the row's
// absmax (a warp reduction), the two divisions, and 128 bytes per row go out.  Returns false if a wait ran out.
template<int MP, bool OUT_F32, int NG, int RB, int CB>
__device__ __forceinline__ bool reduce_split_groups(const SplitGroup (&g)[NG],
                                                    uint32_t* __restrict__ partials,
                                                    void* __restrict__ C_out,
                                                    float* __restrict__ C_s,
                                                    int                M,
                                                    int                N,
                                                    int                lane,
                                                    volatile uint32_t* abort_flag,
                                                    uint32_t*          status)
{
  // (no integer division anywhere in here: a 32-bit division is a dependent chain of ~150 clk, and a dozen of
  // them in a single warp's critical path cost more than the memory round trips)
  constexpr int PW = deccfg::reduce_warps(false);  // warps per contributor that take part
  int max_cnt = 0;
#pragma unroll
  for (int k = 0; k < NG; ++k) {
    max_cnt = g[k].mine ? max(max_cnt, g[k].cnt) : max_cnt;
  }
  for (int pass = 0;; ++pass) {
    // first row of this pass in either group; rows ascend with r, so nothing is left when both are beyond M
    bool more = false;
#pragma unroll
    for (int k = 0; k < NG; ++k) {
      more = more || (g[k].mine && g[k].gw + pass * RB * PW * g[k].cnt < M);
    }
    if (!more) {
      break;
    }
    float4 sum[NG][RB];
#pragma unroll
    for (int k = 0; k < NG; ++k) {
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        sum[k][r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
    for (int cb = 0; cb * CB < max_cnt; ++cb) {
      uint32_t off[NG][RB][CB];  // word offset into the scratch; NONE: nothing to read for this (group, row, contributor)
      constexpr uint32_t NONE = 0xffffffffu;
#pragma unroll
      for (int k = 0; k < NG; ++k) {
#pragma unroll
        for (int j = 0; j < CB; ++j) {
          const int  jj   = cb * CB + j;
          const bool c_ok = g[k].mine && jj < g[k].cnt;
          const int  c    = g[k].c_lo + (c_ok ? jj : 0);
          // the group's first contributor reached it at K-block 0 (slot 1), the others began inside it (slot 0)
          const int  sl   = c * 2 + (jj == 0 ? 1 : 0);
#pragma unroll
          for (int r = 0; r < RB; ++r) {
            const int m  = g[k].gw + (pass * RB + r) * PW * g[k].cnt;
            off[k][r][j] = (c_ok && m < M) ? (uint32_t)((sl * MP + m) * 128 + lane * 4) : NONE;
          }
        }
      }
      uint4              t[NG][RB][CB];
      unsigned long long t0    = 0;
      uint32_t           spins = 0;
      for (;;) {
        bool landed = true;
#pragma unroll
        for (int k = 0; k < NG; ++k) {
#pragma unroll
          for (int r = 0; r < RB; ++r) {
#pragma unroll
            for (int j = 0; j < CB; ++j) {
              if (off[k][r][j] != NONE) {
                t[k][r][j] = ld_partial4(partials + off[k][r][j]);
              }
            }
          }
        }
#pragma unroll
        for (int k = 0; k < NG; ++k) {
#pragma unroll
          for (int r = 0; r < RB; ++r) {
#pragma unroll
            for (int j = 0; j < CB; ++j) {
              if (off[k][r][j] != NONE) {
                landed = landed && t[k][r][j].x != 0u && t[k][r][j].y != 0u && t[k][r][j].z != 0u && t[k][r][j].w != 0u;
              }
            }
          }
        }
#ifdef LLMMM_PROFILE
        if (threadIdx.x == (deccfg::EPI_WARP0 + deccfg::promo_warps(MP)) * 32 && pass == 0 && cb == 0 && spins == 0) {
          g_prof_cta[blockIdx.x][6] = global_timer_ns();  // first poll has returned
        }
#endif
        if (__all_sync(0xffffffffu, landed)) {
#ifdef LLMMM_PROFILE
          if (threadIdx.x == (deccfg::EPI_WARP0 + deccfg::promo_warps(MP)) * 32 && pass == 0 && cb == 0) {
            g_prof_cta[blockIdx.x][10] = global_timer_ns();  // first batch complete
            g_prof_cta[blockIdx.x][11] = spins + 1;          // polls it took (a count, not a time)
          }
#endif
          break;
        }
        ++spins;
        if ((spins & 0x7) == 0) {
          if (*abort_flag) {
            return false;
          }
          const unsigned long long now = global_timer_ns();
          if (t0 == 0) {
            t0 = now;
          }
          else if (now - t0 > WAIT_LIMIT_NS) {
            *abort_flag = DEV_WAIT_SPLITK;
            atomicCAS(status, 0u, (uint32_t)DEV_WAIT_SPLITK);
            return false;
          }
        }
      }
#pragma unroll
      for (int k = 0; k < NG; ++k) {
#pragma unroll
        for (int j = 0; j < CB; ++j) {  // ascending CTA order: the result does not depend on timing
#pragma unroll
          for (int r = 0; r < RB; ++r) {
            if (off[k][r][j] != NONE) {
              // consumed: the words go back to zero for the next launch
              __stcg(reinterpret_cast<uint4*>(partials + off[k][r][j]), make_uint4(0u, 0u, 0u, 0u));
              sum[k][r].x += decode_partial(t[k][r][j].x);
              sum[k][r].y += decode_partial(t[k][r][j].y);
              sum[k][r].z += decode_partial(t[k][r][j].z);
              sum[k][r].w += decode_partial(t[k][r][j].w);
            }
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < NG; ++k) {
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        const int m = g[k].gw + (pass * RB + r) * PW * g[k].cnt;
        if (!g[k].mine || m >= M) {
          continue;
        }
        store_group_row<OUT_F32>(sum[k][r], m, g[k].nb, C_out, C_s, M, N, lane);
      }
    }
  }
  return true;
}

// CLUSTER = false: stream-K over all weight blocks, partial tiles through the caller's scratch (above).
// CLUSTER = true : one thread-block cluster per output group; CTA r of the C in the cluster takes the r-th
//   slice of the group's K range, and the partial tiles are added through distributed shared memory as a
//   reduce-scatter: each CTA stages its partial tile in its own idle TMA ring; after a cluster barrier it sends
//   every other CTA that CTA's share of the rows (bulk copies between shared memories, completion counted on the
//   receiver's barrier), and every CTA adds the partials of its rows in rank order, quantises and stores them,
//   one warp per row; a last cluster barrier keeps everybody until all copies are done.  No scratch, no atomics, no global round trips; used when
//   the groups times a cluster size of 2-7 fill the GPU.
template<int MP, bool OUT_F32, bool CLUSTER>
__global__ void __launch_bounds__(deccfg::threads(MP, CLUSTER), deccfg::ctas_per_sm(MP, CLUSTER)) fp8_decode_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                        const __grid_constant__ CUtensorMap tm_x,
                                                                        const float* __restrict__ A_s,
                                                                        const float* __restrict__ B_s,
                                                                        void* __restrict__ C_out,
                                                                        float* __restrict__ C_s,
                                                                        int       M,
                                                                        int       N,
                                                                        int       K,
                                                                        uint32_t* partials,
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
  PROF_CTA(0);

  const int       KB      = K / BK;
  const uint32_t  U       = (uint32_t)(N / 128) * (uint32_t)KB;  // the launcher keeps U * 256 below 2^31
  const uint32_t  G       = gridDim.x;
  uint32_t        c_size  = 1, c_rank = 0, red_rows = MP;  // (cluster kernel: rows of the group a CTA owns, at most)
  // A CTA works through two ranges of units, [u_begin, u_end) and then [v_begin, v_end).  Stream-K kernel with at
  // least as many output groups as CTAs: every CTA takes floor(groups / G) whole groups (the second range, finished
  // in place), and only the groups that are left over are cut evenly among the CTAs (the first range: their partial
  // tiles are published early and added up by the reduction warps while the second range streams); with fewer groups
  // than CTAs everything is "left over".  Cluster kernel: one slice of one group, no second range.
  uint32_t        u_begin, u_end, v_begin = 0, v_end = 0;
  // the units that are cut: [tail_base, tail_base + tail_units), among the first tail_ctas CTAs (all of them, unless
  // there are fewer such units than CTAs: every CTA that takes part gets at least one)
  uint32_t        tail_base = 0, tail_units = U, tail_ctas = G;
  if constexpr (CLUSTER) {
    asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(c_size));
    c_rank = cluster_ctarank();
    const uint32_t group = blockIdx.x / c_size;
    red_rows = ((uint32_t)M + c_size - 1) / c_size;
    u_begin = group * (uint32_t)KB + (c_rank * (uint32_t)KB) / c_size;
    u_end   = group * (uint32_t)KB + ((c_rank + 1) * (uint32_t)KB) / c_size;
  }
  else {
    const uint32_t whole_units = ((uint32_t)(N / 128) / G) * (uint32_t)KB;  // per CTA
    tail_base  = G * whole_units;
    tail_units = U - tail_base;
    v_begin    = blockIdx.x * whole_units;
    v_end      = v_begin + whole_units;
    tail_ctas  = tail_units < G ? tail_units : G;
    u_begin    = tail_base + (blockIdx.x < tail_ctas ? (blockIdx.x * tail_units) / tail_ctas : 0u);
    u_end      = tail_base + (blockIdx.x < tail_ctas ? ((blockIdx.x + 1) * tail_units) / tail_ctas : 0u);
  }
  const uint32_t len0 = u_end - u_begin;          // units of the first range
  const uint32_t run  = len0 + (v_end - v_begin);  // units of this CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->part_full[s], 1);
      mbar_init(&bars->part_empty[s], promo_warps(MP));
    }
    mbar_init(&bars->red, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc<L::TMEM_COLS>(&bars->tmem_base);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // Set-up (barriers, tensor memory, descriptor prefetch) touched no global memory: it may overlap the tail
  // of the previous kernel on the stream, and the next kernel may begin its own set-up from here on.
  pdl_launch_dependents();
  if (warp != 0) {
    pdl_wait();  // warp 0 waits below, as a whole: a waiting lane holds up the other lanes of its warp
  }
  PROF_CTA(1);

  // The reduction of split groups wants as many loads in flight as registers allow: the control warpgroup hands
  // registers over to the promotion warpgroups.
  if (warp < EPI_WARP0) {
    setmaxnreg_dec<REGS_CTRL>();
  }
  else if (warp < EPI_WARP0 + promo_warps(MP)) {
    if constexpr (CLUSTER || MP <= 16) {  // (the other form keeps the 128 registers it was launched with)
      setmaxnreg_inc<regs_promo(MP, CLUSTER)>();
    }
  }
  else {
    setmaxnreg_inc<regs_reduce(MP)>();
  }
  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    const uint64_t pol_w = policy_evict_first();  // weights are read once
    const uint64_t pol_x = policy_evict_last();   // activations are re-read by every CTA
    // walks the CTA's units in order and calls body(it, nb, kb) until it returns false
    auto walk = [&](auto&& body) {
      uint32_t it = 0;
      for (int r = 0; r < 2; ++r) {
        const uint32_t b = r == 0 ? u_begin : v_begin, e = r == 0 ? u_end : v_end;
        if (b >= e) {
          continue;
        }
        int nb = (int)(b / (uint32_t)KB), kb = (int)(b % (uint32_t)KB);
        for (uint32_t u = b; u < e; ++u, ++it, ++kb) {
          if (kb == KB) {
            kb = 0;
            ++nb;
          }
          if (!body(it, nb, kb)) {
            return;
          }
        }
      }
    };
    // Weights the caller declared static (llmmm_set_static_weights) do not depend on the previous kernel
    // of the stream: the first ring of weight tiles is requested before waiting for that kernel, the
    // activation tiles of the same stages after it.
    uint32_t early = 0;
    if (lane == 0 && early_weights) {
      walk([&](uint32_t it, int nb, int kb) {
        if (it >= (uint32_t)L::STAGES) {
          return false;
        }
        mbar_arrive_expect_tx(&bars->full[it], W_BYTES + L::X_BYTES);
        tma_load_2d_hint(smem + L::OFF_W + it * W_BYTES, &tm_w, &bars->full[it], kb * BK, nb * 128, pol_w);
        early = it + 1;
        return true;
      });
    }
    __syncwarp();
    pdl_wait();
    if (lane == 0) {
      walk([&](uint32_t it, int nb, int kb) {
        const uint32_t s  = it % L::STAGES;
        const uint32_t ph = (it / L::STAGES) & 1;
        if (it >= early) {
          mbar_wait(&bars->part_full[s], ph ^ 1, DEV_WAIT_SMEM_EMPTY, abort_flag, status);
          mbar_arrive_expect_tx(&bars->full[s], W_BYTES + L::X_BYTES);
          tma_load_2d_hint(smem + L::OFF_W + s * W_BYTES, &tm_w, &bars->full[s], kb * BK, nb * 128, pol_w);
        }
        tma_load_2d_hint(smem + L::OFF_X + s * L::X_BYTES, &tm_x, &bars->full[s], kb * BK, 0, pol_x);
        return true;
      });
    }
    if constexpr (CLUSTER) {
      __syncwarp();
      cluster_sync_all();  // every CTA's ring is idle
      cluster_sync_all();  // all partial rows have been delivered
    }
  }
  else if (warp < EPI_WARP0) {
    // --------------------------------------------- three MMA issuers ------
    // Warps 1, 2 and 3 take every third K-block of the run; each K-block has its own ring slot and
    // tensor-memory partial stage, so the threads never touch the same barrier phase.
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*e4m3*/ 0, 0, 0, 0, 128, MP);
      for (uint32_t it = (uint32_t)(warp - 1); it < run; it += 3) {
        const uint32_t s  = it % L::STAGES;
        const uint32_t ph = (it / L::STAGES) & 1;
        mbar_wait(&bars->part_empty[s], ph ^ 1, DEV_WAIT_TMEM_EMPTY, abort_flag, status);
        mbar_wait(&bars->full[s], ph, DEV_WAIT_SMEM_FULL, abort_flag, status);
        if (it == 0) {
          PROF_CTA(2);
        }
        tc_fence_after_sync();
        const uint64_t dw = make_smem_desc_sw128(smem_u32(smem + L::OFF_W + s * W_BYTES), 0, 1024);
        const uint64_t dx = make_smem_desc_sw128(smem_u32(smem + L::OFF_X + s * L::X_BYTES), 0, 1024);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          tc_mma_f8(tmem_base + s * L::PART_COLS, dw + (uint64_t)((kk * UMMA_K) >> 4), dx + (uint64_t)((kk * UMMA_K) >> 4), idesc, kk != 0);
        }
        tc_commit(&bars->part_full[s]);
      }
      if (warp == 1) {
        PROF_CTA(3);
      }
    }
    if constexpr (CLUSTER) {
      __syncwarp();
      cluster_sync_all();
      cluster_sync_all();
    }
  }
  else if (warp < EPI_WARP0 + promo_warps(MP)) {
    // ------------------------------------------- promotion + epilogue ----
    constexpr int  PW      = promo_warps(MP);      // promotion warps
    constexpr int  PT      = 32 * PW;              // promotion threads
    constexpr int  MPH     = MP / (PW / 4);        // activation columns (= output rows) per thread
    const int      quarter = warp & 3;             // tensor-memory lane quarter this warp may read
    const int      ew      = warp - EPI_WARP0;     // 0..PW-1
    const int      row0    = (ew >> 2) * MPH;      // first output row this thread accumulates
    const int      n_local = quarter * 32 + lane;  // output column inside the group == TMEM lane
    const int      et      = threadIdx.x - EPI_WARP0 * 32;  // 0..PT-1
    const uint32_t t_lane  = (uint32_t)(quarter * 32) << 16;
    uint32_t       it      = 0;

    // Scale products of the run, CHUNK K-blocks at a time: thread `et` fetches elements et, et + PT, ... of
    // the [CHUNK][MP] chunk (A_s[kb, m] and B_s[nb, kb]: the latter is simply B_s[u] for unit u), multiplies
    // (one fp32 rounding of each scale product, as in the reference) and keeps them in registers until the
    // chunk before has been used up.  All loads of a chunk are in flight together; for runs of up to CHUNK
    // K-blocks there is exactly one L2 round trip, hidden behind the first operand tiles.
    constexpr int CH = L::CHUNK;
    constexpr int SE = CH * MP / PT;  // elements per thread
    static_assert(SE * PT == CH * MP, "a chunk of scale products must divide among the promotion threads");
    float*        sc = reinterpret_cast<float*>(smem + L::OFF_SC);
    float         st[SE];
    auto fetch_chunk = [&](uint32_t chunk) {
#pragma unroll
      for (int i = 0; i < SE; ++i) {
        const uint32_t e   = (uint32_t)et + (uint32_t)PT * (uint32_t)i;
        const uint32_t itx = chunk * CH + e / MP;
        const int      m   = (int)(e % MP);
        float          v   = 0.0f;
        if (itx < run && m < M) {
          const uint32_t uu = itx < len0 ? u_begin + itx : v_begin + (itx - len0);
          v = __fmul_rn(__ldg(A_s + (size_t)(uu % (uint32_t)KB) * M + m), __ldg(B_s + uu));
        }
        st[i] = v;
      }
    };
    auto store_chunk = [&]() {
#pragma unroll
      for (int i = 0; i < SE; ++i) {
        sc[et + PT * i] = st[i];
      }
    };
    fetch_chunk(0);
    store_chunk();
    epilogue_bar_sync<PT>();
    if (run > (uint32_t)CH) {
      fetch_chunk(1);
    }

    for (int range = 0; range < (CLUSTER ? 1 : 2); ++range) {
    uint32_t       u     = range == 0 ? u_begin : v_begin;
    const uint32_t r_end = range == 0 ? u_end : v_end;
    bool           first = range == 0;  // a cluster CTA runs its one segment even if it is empty: it owes two cluster barriers
    while (u < r_end || (CLUSTER && first)) {
      first = false;
      const int      nb   = (int)(u / (uint32_t)KB);
      const int      kb0  = (int)(u % (uint32_t)KB);
      const uint32_t left = r_end - u;
      const int      kb1  = (left < (uint32_t)(KB - kb0)) ? kb0 + (int)left : KB;
      const bool     whole = (kb0 == 0 && kb1 == KB);

      float acc[MPH];  // output rows row0 .. row0 + MPH - 1 of column n_local
#pragma unroll
      for (int i = 0; i < MPH; ++i) {
        acc[i] = 0.0f;
      }
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const uint32_t p  = it % L::STAGES;
        const uint32_t pp = (it / L::STAGES) & 1;
        if (it != 0 && it % CH == 0) {
          // the next chunk's products are in `st`: swap them in once everybody is done with the old ones
          epilogue_bar_sync<PT>();
          store_chunk();
          epilogue_bar_sync<PT>();
          if ((it / CH + 1) * CH < run) {
            fetch_chunk(it / CH + 1);
          }
        }
        // One promotion warp has a scheduler to itself: nothing hides a shared-memory latency in front of every four
        // FMAs.  The scale products of the first half of the rows are therefore fetched before the wait for the
        // partial, those of the second half while the first half is being worked on.
        constexpr int H4   = MPH / 8;  // float4 values per half
        const float4* srow = reinterpret_cast<const float4*>(sc + (it % CH) * MP + row0);
        float4        s_lo[H4], s_hi[H4];
#pragma unroll
        for (int i = 0; i < H4; ++i) {
          s_lo[i] = srow[i];  // the same address in every lane: a broadcast
        }
        PROF_KB(0);
        mbar_wait(&bars->part_full[p], pp, DEV_WAIT_TMEM_FULL, abort_flag, status);
        PROF_KB(1);
        tc_fence_after_sync();
        // the partial goes to registers and the stage is handed back as soon as its last column has been read,
        // before the arithmetic on it
        uint32_t v[MPH];
#pragma unroll
        for (int c = 0; c < MPH / 16; ++c) {
          tmem_ld_32x32b_x16(tmem_base + p * L::PART_COLS + t_lane + row0 + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&v[c * 16]));
        }
#pragma unroll
        for (int i = 0; i < H4; ++i) {
          s_hi[i] = srow[H4 + i];
        }
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->part_empty[p]);
        }
        PROF_KB(2);
#pragma unroll
        for (int i = 0; i < H4; ++i) {
          acc[4 * i]     = __fmaf_rn(__uint_as_float(v[4 * i]), s_lo[i].x, acc[4 * i]);
          acc[4 * i + 1] = __fmaf_rn(__uint_as_float(v[4 * i + 1]), s_lo[i].y, acc[4 * i + 1]);
          acc[4 * i + 2] = __fmaf_rn(__uint_as_float(v[4 * i + 2]), s_lo[i].z, acc[4 * i + 2]);
          acc[4 * i + 3] = __fmaf_rn(__uint_as_float(v[4 * i + 3]), s_lo[i].w, acc[4 * i + 3]);
        }
#pragma unroll
        for (int i = 0; i < H4; ++i) {
          const int m = 4 * (H4 + i);
          acc[m]     = __fmaf_rn(__uint_as_float(v[m]), s_hi[i].x, acc[m]);
          acc[m + 1] = __fmaf_rn(__uint_as_float(v[m + 1]), s_hi[i].y, acc[m + 1]);
          acc[m + 2] = __fmaf_rn(__uint_as_float(v[m + 2]), s_hi[i].z, acc[m + 2]);
          acc[m + 3] = __fmaf_rn(__uint_as_float(v[m + 3]), s_hi[i].w, acc[m + 3]);
        }
        PROF_KB(3);
      }
      u += (uint32_t)(kb1 - kb0);
      if (it >= run && ew == 0) {
        PROF_CTA(4);
      }

      bool finish = whole;
      if constexpr (CLUSTER) {
        // Reduce-scatter through distributed shared memory.  CTA o of the cluster owns rows [o R, (o+1) R) of the
        // group, R = ceil(M / c_size).  Every CTA puts its partial tile into its own idle ring (stage[row][n]) and
        // sends each other CTA that CTA's rows with one bulk copy (shared memory to the peer's shared memory,
        // completion counted in bytes on the peer's barrier); plain remote stores are held to one in flight per
        // warp and took 6 us for 64 rows.  Then one warp per owned row adds the partials in rank order.
        float*         stage   = reinterpret_cast<float*>(smem + L::OFF_W);  // [MP][128]
        float*         rcv     = stage + MP * 128;                           // [c_size][R][128]
        const uint32_t R       = red_rows;
        const uint32_t my_row0 = c_rank * R;
        const uint32_t my_rows = (uint32_t)M > my_row0 ? min(R, (uint32_t)M - my_row0) : 0u;
#pragma unroll
        for (int i = 0; i < MPH; ++i) {
          if (row0 + i < M) {
            stage[(row0 + i) * 128 + n_local] = acc[i];  // (this CTA's MMAs are all done: its ring is idle)
          }
        }
        fence_proxy_async_smem();  // the bulk copies below read what was just written
        if (et == 0) {
          mbar_arrive_expect_tx(&bars->red, (c_size - 1) * my_rows * 512u);
        }
        cluster_sync_all();  // every CTA's ring is idle and its staging tile complete
        if (ew == 0) {
          PROF_CTA(5);
        }
        if (ew == 0 && (uint32_t)lane < c_size) {  // one lane per destination
          const uint32_t o    = (uint32_t)lane;
          const uint32_t rows = (uint32_t)M > o * R ? min(R, (uint32_t)M - o * R) : 0u;
          if (o != c_rank && rows != 0) {
            bulk_copy_to_peer(mapa_shared(smem_u32(rcv + (size_t)c_rank * R * 128), o), stage + (size_t)o * R * 128, rows * 512u,
                              mapa_shared(smem_u32(&bars->red), o));
          }
        }
        __syncwarp();
        if (my_rows != 0) {
          mbar_wait(&bars->red, 0, DEV_WAIT_SPLITK, abort_flag, status);
        }
        // Nobody may leave while a copy can still read its staging tile or write its ring: everybody says here
        // that its own rows have arrived, and waits for the others only after its arithmetic.
        cluster_arrive();
        if (ew == 0) {
          PROF_CTA(6);
        }
        for (uint32_t q = (uint32_t)ew; q < my_rows; q += (uint32_t)PW) {
          float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          for (uint32_t rr = 0; rr < c_size; ++rr) {  // fixed order: the result does not depend on timing
            const float* src = rr == c_rank ? stage + (size_t)(my_row0 + q) * 128 : rcv + ((size_t)rr * R + q) * 128;
            const float4 t   = reinterpret_cast<const float4*>(src)[lane];
            sum.x += t.x;
            sum.y += t.y;
            sum.z += t.z;
            sum.w += t.w;
          }
          store_group_row<OUT_F32>(sum, (int)(my_row0 + q), nb, C_out, C_s, M, N, lane);
        }
        if (ew == 0) {
          PROF_CTA(7);
        }
        cluster_wait();
        finish = false;
      }
      else if (!whole) {
        // publish this CTA's partial tile as flagged words; the reduction warps take it from there
        const int slot = blockIdx.x * 2 + (kb0 == 0 ? 1 : 0);  // run begins inside the group -> slot 0
        uint32_t* dst  = partials + (size_t)slot * (MP * 128);
#pragma unroll
        for (int i = 0; i < MPH; ++i) {
          if (row0 + i < M) {
            st_partial(dst + (row0 + i) * 128 + n_local, acc[i]);
          }
        }
      }

      if (finish) {
        const size_t n_glob = (size_t)nb * 128 + n_local;
        if constexpr (OUT_F32) {
          float* C = reinterpret_cast<float*>(C_out);
#pragma unroll
          for (int i = 0; i < MPH; ++i) {
            if (row0 + i < M) {
              C[(size_t)(row0 + i) * N + n_glob] = acc[i];
            }
          }
        }
        else {
          // group absmax over the 128 lanes: one warp-wide integer max per row (the bit pattern of a
          // non-negative float orders like the float), then the 4 lane quarters through shared memory
#pragma unroll
          for (int i = 0; i < MPH; ++i) {
            if (row0 + i < M) {
              const uint32_t a = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(acc[i])));
              if (lane == 0) {
                bars->amax[quarter][row0 + i] = __uint_as_float(a);
              }
            }
          }
          epilogue_bar_sync<PT>();
          if (ew == 0) {
            PROF_CTA(12);
          }
          // thread i finishes row i's absmax and does the two divisions once for everybody
          if (et < M) {
            const float amax = fmaxf(fmaxf(bars->amax[0][et], bars->amax[1][et]), fmaxf(bars->amax[2][et], bars->amax[3][et]));
            bars->inv[et]    = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
            C_s[(size_t)nb * M + et] = __fdiv_rn(amax, 448.0f);
          }
          epilogue_bar_sync<PT>();
          if (ew == 0) {
            PROF_CTA(13);
          }
          uint8_t* C = reinterpret_cast<uint8_t*>(C_out);
#pragma unroll
          for (int i = 0; i < MPH; ++i) {
            if (row0 + i < M) {
              C[(size_t)(row0 + i) * N + n_glob] = (uint8_t)__nv_cvt_float_to_fp8(acc[i] * bars->inv[row0 + i], __NV_SATFINITE, __NV_E4M3);
            }
          }
          epilogue_bar_sync<PT>();  // bars->amax and bars->inv are reused by the next segment
          if (ew == 0) {
            PROF_CTA(14);
          }
        }
      }
    }
    }  // range

    if (ew == 0) {
      PROF_CTA(8);
    }
  }
  else {
    // ------------------------------------------- reduce-scatter of the split groups ----
    // (stream-K kernel only.)  The output groups that were cut among CTAs are added up by a warpgroup of their own,
    // beside the promotion warps: a CTA's cut segments lie in its first range, so their partial tiles are
    // published early, and when whole groups follow (second range) the sums are finished long before the CTA's
    // stream ends; otherwise these warps wait, politely (one word per contributor, with a pause between polls),
    // for the other contributors to get there.
    // Group nb was cut among CTAs c_lo..c_hi.  Its M rows are dealt out to the RW * (c_hi - c_lo + 1) reduction
    // warps of those CTAs: warp w of contributor j takes rows RW j + w, RW j + w + RW cnt, ...  A warp reads
    // (bounded) until the words of every contributor have landed -- all CTAs of the grid are resident, the
    // grid is never larger than the SM count -- and reduces its rows of both groups this CTA took part in
    // (reduce_split_groups).
    if constexpr (!CLUSTER) {
      constexpr int RW = reduce_warps(false);
      const int     rw = warp - EPI_WARP0 - promo_warps(MP);  // 0..RW-1
      // the cut segments of this CTA's first range: at most its first and its last one
      int pend_nb0 = 0, pend_nb1 = 0;
      int n_pend = 0;
      for (uint32_t u = u_begin; u < u_end;) {
        const int      nb   = (int)(u / (uint32_t)KB);
        const int      kb0  = (int)(u % (uint32_t)KB);
        const uint32_t left = u_end - u;
        const int      kb1  = (left < (uint32_t)(KB - kb0)) ? kb0 + (int)left : KB;
        if (!(kb0 == 0 && kb1 == KB)) {
          if (n_pend == 0) {
            pend_nb0 = nb;
          }
          else {
            pend_nb1 = nb;
          }
          ++n_pend;
        }
        u += (uint32_t)(kb1 - kb0);
      }
      if (n_pend > 0) {
        if (rw == 0) {
          PROF_CTA(5);
        }
        // first and last contributor of both groups: four divisions, one per lane
        uint32_t q = 0;
        if (lane < 4) {
          const uint32_t nbq = (uint32_t)(lane < 2 ? pend_nb0 : pend_nb1);
          // (cut groups lie in the tail: their units count from tail_base and are dealt among all CTAs)
          q = (uint32_t)cta_of_unit(((lane & 1) ? (nbq + 1) * (uint32_t)KB - 1 : nbq * (uint32_t)KB) - tail_base, tail_ctas, tail_units);
        }
        SplitGroup g[2];
        int        max_cnt = 0;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          g[k].nb   = k == 0 ? pend_nb0 : pend_nb1;
          g[k].c_lo = (int)__shfl_sync(0xffffffffu, q, 2 * k);
          g[k].cnt  = (int)__shfl_sync(0xffffffffu, q, 2 * k + 1) - g[k].c_lo + 1;
          g[k].gw   = RW * ((int)blockIdx.x - g[k].c_lo) + rw;
          g[k].mine = k < n_pend && g[k].gw < M;  // more warps than rows: some have none
          if (g[k].mine) {
            max_cnt = max(max_cnt, g[k].cnt);
          }
        }
        bool alive = true;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (alive && g[k].mine) {
            alive = wait_contributors<MP>(g[k], partials, lane, abort_flag, status);
          }
        }
        if (alive && (g[0].mine || g[1].mine)) {
          if constexpr (MP <= 16) {
            // (96 registers per thread: eight partial rows of 16 bytes per lane in flight)
            if (max_cnt <= 2) {
              reduce_split_groups<MP, OUT_F32, 2, 2, 2>(g, partials, C_out, C_s, M, N, lane, abort_flag, status);
            }
            else if (max_cnt <= 4) {
              reduce_split_groups<MP, OUT_F32, 2, 1, 4>(g, partials, C_out, C_s, M, N, lane, abort_flag, status);
            }
            else {
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                if (g[k].mine) {
                  const SplitGroup one[1] = {g[k]};
                  reduce_split_groups<MP, OUT_F32, 1, 1, 8>(one, partials, C_out, C_s, M, N, lane, abort_flag, status);
                }
              }
            }
          }
          else if (max_cnt <= 2) {
            reduce_split_groups<MP, OUT_F32, 2, 4, 2>(g, partials, C_out, C_s, M, N, lane, abort_flag, status);
          }
          else if (max_cnt <= 4) {
            reduce_split_groups<MP, OUT_F32, 2, 2, 4>(g, partials, C_out, C_s, M, N, lane, abort_flag, status);
          }
          else if (max_cnt <= 8) {
            reduce_split_groups<MP, OUT_F32, 2, 1, 8>(g, partials, C_out, C_s, M, N, lane, abort_flag, status);
          }
          else {
            // many contributors with one or two K-blocks each (the left-over groups of a shape with more groups
            // than CTAs): one group after the other, 24 contributors' rows in flight
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              if (g[k].mine) {
                const SplitGroup one[1] = {g[k]};
                reduce_split_groups<MP, OUT_F32, 1, 1, 24>(one, partials, C_out, C_s, M, N, lane, abort_flag, status);
              }
            }
          }
        }
        if (rw == 0) {
          PROF_CTA(7);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<L::TMEM_COLS>(tmem_base);
    PROF_CTA(9);
  }
}

#ifdef LLMMM_PROFILE
// Profiling build only (python -m llmmm_b200.build --profile): prints the phase stamps of the last decode launch.
extern "C" void llmmm_profile_dump_decode()
{
  // (slot 11 is a count, printed below; 12-14: the last in-place finish of a whole group)
  static const char* names[15] = {"entry", "released", "first operands", "MMAs issued", "promotion done", "published",
                                  "first poll back", "rows reduced", "roles done", "TMEM freed", "first batch in", "",
                                  "row maxima met", "scales ready", "group stored"};
  static unsigned long long c[256][16];
  cudaMemcpyFromSymbol(c, g_prof_cta, sizeof(c));
  unsigned long long t0 = ~0ull, rel = ~0ull;
  int                n  = 0;
  for (int i = 0; i < 256; ++i) {
    if (c[i][0] == 0) {
      continue;
    }
    ++n;
    t0  = c[i][0] < t0 ? c[i][0] : t0;
    rel = c[i][1] < rel ? c[i][1] : rel;
  }
  if (n == 0) {
    printf("no decode launch recorded\n");
    return;
  }
  printf("decode launch, %d CTAs; ns after the first release (min / mean / max over CTAs):\n", n);
  for (int k = 0; k < 15; ++k) {
    if (k == 11) {
      continue;
    }
    double             sum = 0;
    long long          mn = 1ll << 62, mx = -(1ll << 62);
    int                cnt = 0;
    for (int i = 0; i < 256; ++i) {
      if (c[i][0] == 0 || c[i][k] == 0) {
        continue;
      }
      const long long d = (long long)(c[i][k] - rel);
      sum += (double)d;
      mn = d < mn ? d : mn;
      mx = d > mx ? d : mx;
      ++cnt;
    }
    if (cnt) {
      printf("  %-18s %7lld %9.0f %7lld  (%d CTAs)\n", names[k], mn, sum / cnt, mx, cnt);
    }
  }
  {
    double polls = 0;
    int    cnt   = 0, mx = 0;
    for (int i = 0; i < 256; ++i) {
      if (c[i][0] != 0 && c[i][11] != 0) {
        polls += (double)c[i][11];
        mx = (int)c[i][11] > mx ? (int)c[i][11] : mx;
        ++cnt;
      }
    }
    if (cnt) {
      printf("  polls until the first batch was complete: mean %.1f, max %d\n", polls / cnt, mx);
    }
  }
  {
    unsigned long long kb[8][4];
    cudaMemcpyFromSymbol(kb, g_prof_kb, sizeof(kb));
    printf("  CTA 0, first promotion warp, per K-block (ns after release): waiting / partial seen / read / done\n");
    for (int i = 0; i < 8; ++i) {
      if (kb[i][0]) {
        printf("    %d: %lld %lld %lld %lld\n", i, (long long)(kb[i][0] - rel), (long long)(kb[i][1] - rel), (long long)(kb[i][2] - rel),
               (long long)(kb[i][3] - rel));
      }
    }
    static unsigned long long zkb[8][4];
    cudaMemcpyToSymbol(g_prof_kb, zkb, sizeof(zkb));
  }
  static unsigned long long zero[256][16];
  cudaMemcpyToSymbol(g_prof_cta, zero, sizeof(zero));
}
#endif

// ------------------------------------------------------------ host side ---

std::atomic<int> g_static_weights{0};  // llmmm_set_static_weights()

namespace {
Workspace  g_ws[64];
std::mutex g_ws_mutex;

int padded_m(int M)
{
  return M <= 16 ? 16 : (M <= 32 ? 32 : 64);
}
}  // namespace

// Partial tiles of the stream-K kernel: two slots per CTA of M (padded) x 128 self-announcing 32-bit words.
static size_t decode_partial_bytes(int M)
{
  return (size_t)deccfg::MAX_CTAS * 2 * padded_m(M) * 128 * sizeof(uint32_t);
}

// The decode kernel's partial tiles lie behind the split tiles of the pair kernels (whose region is never
// zero): they must be all zero between launches.
size_t decode_workspace_bytes(int M)
{
  return split_workspace_bytes() + decode_partial_bytes(M);
}

namespace {
thread_local Workspace t_ws;
thread_local bool      t_ws_bound = false;
}  // namespace

Workspace registered_workspace(int device)
{
  if (t_ws_bound) {
    return t_ws;
  }
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  return g_ws[device];
}

bool thread_workspace_bound()
{
  return t_ws_bound;
}

ScopedWorkspace::ScopedWorkspace(void* ptr, size_t bytes): prev_(t_ws), prev_bound_(t_ws_bound)
{
  t_ws.ptr   = ptr;
  t_ws.bytes = ptr ? bytes : 0;
  t_ws_bound = true;
}

ScopedWorkspace::~ScopedWorkspace()
{
  t_ws       = prev_;
  t_ws_bound = prev_bound_;
}

int check_workspace_arg(const void* ptr, size_t bytes)
{
  if (ptr == nullptr) {
    return bytes == 0 ? LLMMM_OK : set_error(LLMMM_ERR_SHAPE, "a null workspace must have zero bytes");
  }
  if (((uintptr_t)ptr & 255) != 0 || bytes < WS_HEADER_BYTES) {
    return set_error(LLMMM_ERR_SHAPE, "workspace must be 256-byte aligned and at least %zu bytes", WS_HEADER_BYTES);
  }
  return LLMMM_OK;
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
                           uint32_t*         partials,
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
  LLMMM_CUDA_TRY(launch_pdl(fp8_decode_kernel<MP, OUT_F32, false>, dim3((unsigned)G), dim3(threads(MP, false)), L::SMEM_BYTES, stream,
                            1, tm_w, tm_x, A_s, B_s, C, C_s, M, N, K, partials, g_static_weights.load(),
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
  uint32_t* no_partials = nullptr;
  LLMMM_CUDA_TRY(launch_pdl(fp8_decode_kernel<MP, OUT_F32, true>, dim3((unsigned)((N / 128) * cluster)), dim3(threads(MP, true)),
                            L::SMEM_BYTES, stream, (unsigned)cluster, tm_w, tm_x, A_s, B_s, C, C_s, M, N, K, no_partials,
                            g_static_weights.load(), info->status));
  g_launches.fetch_add(1);
  return LLMMM_OK;
}

namespace {
// How many clusters of `size` CTAs of the cluster kernel for activation tiles of `mp` columns the device can hold
// at once (an occupancy query, cached).
template<int MP>
int cluster_capacity_t(const DeviceInfo* info, int size)
{
  using L = DecodeSmem<MP>;
  int clusters = 0;
  if (cudaFuncSetAttribute(fp8_decode_kernel<MP, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM_BYTES)
      == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim            = dim3((unsigned)(size * (info->sm_count / size)));
    cfg.blockDim           = dim3(deccfg::threads(MP, true));
    cfg.dynamicSmemBytes   = L::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = 1;
    if (cudaOccupancyMaxActiveClusters(&clusters, fp8_decode_kernel<MP, false, true>, &cfg) != cudaSuccess) {
      clusters = 0;
    }
  }
  cudaGetLastError();
  return clusters;
}

int cluster_capacity(const DeviceInfo* info, int size, int mp)
{
  static std::mutex mu;
  static int        cache[64][3][9];
  static bool       known[64][3][9];
  const int         slot = mp == 16 ? 0 : (mp == 32 ? 1 : 2);
  std::lock_guard<std::mutex> lock(mu);
  if (!known[info->device][slot][size]) {
    cache[info->device][slot][size] = mp == 16 ? cluster_capacity_t<16>(info, size)
                                               : (mp == 32 ? cluster_capacity_t<32>(info, size) : cluster_capacity_t<64>(info, size));
    known[info->device][slot][size] = true;
  }
  return cache[info->device][slot][size];
}

// Largest allowed cluster size for which every output group gets a resident cluster and every CTA at least
// one K-block; 0 when the cluster path does not apply (then stream-K with scratch is used).
int choose_cluster(const DeviceInfo* info, int M, int N, int K)
{
  const int groups = N / 128, kb = K / 128;
  for (int size = 7; size >= 2; --size) {
    if (kb >= size && groups * size <= info->sm_count && cluster_capacity(info, size, padded_m(M)) >= groups) {
      // worth it only if the clusters occupy at least half of the SMs; otherwise stream-K spreads the weight
      // blocks over all of them
      return (groups * size * 2 >= info->sm_count) ? size : 0;
    }
  }
  return 0;
}

// Choices measured by llmmm_tune (tune_decode below): (device, padded M, N, K) -> cluster size, 0 = stream-K.
std::map<std::array<int, 4>, int> g_plan_table;
std::mutex                        g_plan_mutex;

bool cluster_fits(const DeviceInfo* info, int mp, int N, int K, int size)
{
  const int groups = N / 128, kb = K / 128;
  return kb >= size && groups * size <= info->sm_count && cluster_capacity(info, size, mp) >= groups;
}

bool scratch_fits(const DeviceInfo* info, int M)
{
  const Workspace ws = registered_workspace(info->device);
  return ws.ptr != nullptr && ws.bytes >= decode_workspace_bytes(M);
}

// The cluster size a call gets (0: stream-K): the measured choice if llmmm_tune has seen this (N, K) on this
// device, else the closed-form one.  A measured "stream-K" is ignored while no scratch is registered.
int planned_cluster(const DeviceInfo* info, int M, int N, int K, bool* tuned)
{
  {
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    const auto                  it = g_plan_table.find({info->device, padded_m(M), N, K});
    if (it != g_plan_table.end() && (it->second != 0 || scratch_fits(info, M))) {
      if (tuned != nullptr) {
        *tuned = true;
      }
      return it->second;
    }
  }
  if (tuned != nullptr) {
    *tuned = false;
  }
  return choose_cluster(info, M, N, K);
}
}  // namespace

bool describe_decode_plan(const DeviceInfo* info, int M, int N, int K, char* buf, size_t len)
{
  if (M > 64 || N / 128 > deccfg::MAX_GROUPS || (long long)(N / 128) * (K / 128) * 256 >= (1ll << 31)) {
    return false;
  }
  const int   mp    = padded_m(M);
  bool        tuned = false;
  const int   cluster = planned_cluster(info, M, N, K, &tuned);
  const char* how     = tuned ? "measured by llmmm_tune" : "default rule";
  if (cluster != 0) {
    snprintf(buf, len, "fp8_decode_kernel<%d, cluster>: %d output groups x clusters of %d CTAs, each CTA streams %d or %d of the "
             "%d K-blocks; reduce-scatter through distributed shared memory, no scratch (choice: %s)", mp, N / 128, cluster,
             (K / 128) / cluster, (K / 128 + cluster - 1) / cluster, K / 128, how);
    return true;
  }
  const Workspace ws = registered_workspace(info->device);
  if (ws.ptr == nullptr || ws.bytes < decode_workspace_bytes(M)) {
    return false;  // no scratch: the general kernel runs
  }
  const long long U = (long long)(N / 128) * (K / 128);
  long long       G = info->sm_count < deccfg::MAX_CTAS ? info->sm_count : deccfg::MAX_CTAS;
  G                 = G < U ? G : U;
  const long long whole = (N / 128) / G;              // whole output groups per CTA
  const long long cut   = (N / 128) - whole * G;      // groups cut evenly among all CTAs
  snprintf(buf, len, "fp8_decode_kernel<%d, stream-K>: %lld weight blocks of 128x128 over %lld CTAs (%.1f each): %lld whole output "
           "group(s) per CTA finished in place, %lld group(s) cut evenly among all CTAs, their partial tiles through the registered "
           "scratch and their rows added up by the contributors' reduction warps beside the stream (choice: %s)", mp, U, G, (double)U / (double)G, whole, cut, how);
  return true;
}

namespace {
int noalloc_scratch(const DeviceInfo* info, uint8_t** out);  // (below: the entry point without scratch)
}

int warm_decode_kernels(const DeviceInfo* info)
{
  // touches this module, so that its built-in scratch exists from here on, and looks its address up
  uint8_t* builtin = nullptr;
  if (const int rc = noalloc_scratch(info, &builtin)) {
    return rc;
  }
#define LLMMM_WARM_DECODE(MPV, F32, CL)                                                                                \
  LLMMM_CUDA_TRY(cudaFuncSetAttribute(fp8_decode_kernel<MPV, F32, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                      (int)DecodeSmem<MPV>::SMEM_BYTES));
  LLMMM_WARM_DECODE(16, false, false) LLMMM_WARM_DECODE(16, true, false) LLMMM_WARM_DECODE(16, false, true) LLMMM_WARM_DECODE(16, true, true)
  LLMMM_WARM_DECODE(32, false, false) LLMMM_WARM_DECODE(32, true, false) LLMMM_WARM_DECODE(32, false, true) LLMMM_WARM_DECODE(32, true, true)
  LLMMM_WARM_DECODE(64, false, false) LLMMM_WARM_DECODE(64, true, false) LLMMM_WARM_DECODE(64, false, true) LLMMM_WARM_DECODE(64, true, true)
#undef LLMMM_WARM_DECODE
  for (int size = 2; size <= 7; ++size) {
    for (int mp = 16; mp <= 64; mp *= 2) {
      cluster_capacity(info, size, mp);  // occupancy queries, cached
    }
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
                  cudaStream_t stream,
                  int          force_cluster)
{
  if (M > 64 || N / 128 > deccfg::MAX_GROUPS || (long long)(N / 128) * (K / 128) * 256 >= (1ll << 31)) {
    return -1;
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  const int mp = padded_m(M);
  if (const int cluster = force_cluster >= 0 ? force_cluster : planned_cluster(info, M, N, K, nullptr)) {
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
  uint32_t* partials = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ws.ptr) + split_workspace_bytes());
  if (!thread_workspace_bound() && g_scratch_dirty[info->device].exchange(0) != 0) {
    // a wait ran out in an earlier launch (llmmm_check_status reported it): words may have been left behind
    LLMMM_CUDA_TRY(cudaMemsetAsync(partials, 0, ws.bytes - split_workspace_bytes(), stream));
  }
#define LLMMM_DECODE_CASE(MPV)                                                                                         \
  if (mp == MPV) {                                                                                                     \
    return out_f32 ? launch_decode_t<MPV, true>(A, A_s, B, B_s, C, C_s, M, N, K, partials, info, stream) :             \
                     launch_decode_t<MPV, false>(A, A_s, B, B_s, C, C_s, M, N, K, partials, info, stream);             \
  }
  LLMMM_DECODE_CASE(16)
  LLMMM_DECODE_CASE(32)
  LLMMM_DECODE_CASE(64)
#undef LLMMM_DECODE_CASE
  return -1;
}


// The search behind llmmm_tune for decode-sized FP8 calls on an [N, K] weight (the reference declares
// tune(N, K) on its planned functor and lists auto-tuning as to do: src/mm/fp32/impl.h:20, README.md:22).
// For M = 16, 32 and 64 (the three activation tile widths) every plan that fits is timed with CUDA events on
// a private stream: stream-K through the registered scratch (if one large enough is registered) and
// clusters of 2..7 CTAs per output group.  For 65..128 rows the single-CTA kernel is timed against the pair
// kernel (at M = 128, with the scratch registered, without which the pair kernel has no case there).  Weights rotate over copies that together exceed the L2 cache, as
// they do in a model whose layers are visited in turn.  The winner goes into the plan table.
int tune_decode(const DeviceInfo* info, int N, int K)
{
  if (N < 128 || K < 128 || (N % 128) != 0 || (K % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "N or K are not aligned. (need N%%128==0, K%%128==0; got %d %d)", N, K);
  }
  const bool decode_shape = !(N / 128 > deccfg::MAX_GROUPS || (long long)(N / 128) * (K / 128) * 256 >= (1ll << 31));
  const size_t w_bytes = (size_t)N * K;
  int          copies  = (int)((size_t(256) << 20) / w_bytes) + 1;
  copies               = copies < 2 ? 2 : (copies > 64 ? 64 : copies);
  uint8_t *B = nullptr, *A = nullptr, *C = nullptr;
  float *  B_s = nullptr, *A_s = nullptr, *C_s = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t  e0 = nullptr, e1 = nullptr;
  const size_t bs_bytes = (size_t)(N / 128) * (K / 128) * sizeof(float);
  const size_t as_bytes = (size_t)(K / 128) * 128 * sizeof(float);  // up to 128 rows: the 65..128-row bucket below
  const size_t cs_bytes = (size_t)(N / 128) * 128 * sizeof(float);
  auto cleanup = [&]() {
    cudaFree(B);
    cudaFree(A);
    cudaFree(C);
    cudaFree(B_s);
    cudaFree(A_s);
    cudaFree(C_s);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (stream) cudaStreamDestroy(stream);
  };
  cudaError_t err = cudaMalloc(&B, w_bytes * copies);
  if (err == cudaSuccess) err = cudaMalloc(&A, (size_t)128 * K);
  if (err == cudaSuccess) err = cudaMalloc(&C, (size_t)128 * N);
  if (err == cudaSuccess) err = cudaMalloc(&B_s, bs_bytes);
  if (err == cudaSuccess) err = cudaMalloc(&A_s, as_bytes);
  if (err == cudaSuccess) err = cudaMalloc(&C_s, cs_bytes);
  if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  if (err == cudaSuccess) err = cudaEventCreate(&e0);
  if (err == cudaSuccess) err = cudaEventCreate(&e1);
  // 0x38 is 1.0 in e4m3; a float made of 0x3c bytes is 0.0115: any finite values do, the time does not depend on them
  if (err == cudaSuccess) err = cudaMemsetAsync(B, 0x38, w_bytes * copies, stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(A, 0x38, (size_t)128 * K, stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(B_s, 0x3c, bs_bytes, stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(A_s, 0x3c, as_bytes, stream);
  if (err != cudaSuccess) {
    cleanup();
    cudaGetLastError();
    return set_error(LLMMM_ERR_CUDA, "llmmm_tune needs %zu bytes of temporary device memory: %s", w_bytes * copies,
                     cudaGetErrorString(err));
  }
  int rc = LLMMM_OK;
  // times `copies` launches of one candidate (the first of four passes warms up); < 0 if a launch failed
  auto time_candidate = [&](auto&& launch_one) -> float {
    float best = -1.0f;
    for (int rep = 0; rep < 4 && rc == LLMMM_OK; ++rep) {
      cudaEventRecord(e0, stream);
      for (int c = 0; c < copies && rc == LLMMM_OK; ++c) {
        rc = launch_one(B + (size_t)c * w_bytes);
      }
      cudaEventRecord(e1, stream);
      if (cudaEventSynchronize(e1) != cudaSuccess) {
        rc = set_error(LLMMM_ERR_CUDA, "llmmm_tune: a timed launch failed: %s", cudaGetErrorString(cudaGetLastError()));
      }
      float ms = 0.0f;
      cudaEventElapsedTime(&ms, e0, e1);
      if (rep > 0 && (best < 0.0f || ms < best)) {
        best = ms;
      }
    }
    return rc == LLMMM_OK ? best : -1.0f;
  };
  // 65..128 rows: single-CTA kernel against pair kernel (which needs the scratch to cut its last wave), at M = 128
  {
    const Workspace ws = registered_workspace(info->device);
    if (info->max_pairs >= 1 && ws.ptr != nullptr && ws.bytes >= split_workspace_bytes()) {
      float t[2];
      for (int cand = 0; cand < 2 && rc == LLMMM_OK; ++cand) {
        t_force_mid = cand;
        t[cand]     = time_candidate([&](const uint8_t* w) { return launch_fp8_e4m3(A, A_s, w, B_s, C, C_s, 128, N, K, stream); });
        t_force_mid = -1;
      }
      if (rc == LLMMM_OK && t[0] >= 0.0f && t[1] >= 0.0f) {
        record_mid_choice(info->device, N, K, t[1] < t[0] ? 1 : 0);
      }
    }
  }
  for (int mp = 16; decode_shape && mp <= 64 && rc == LLMMM_OK; mp *= 2) {
    std::vector<int> candidates;
    if (scratch_fits(info, mp)) {
      candidates.push_back(0);
    }
    for (int size = 2; size <= 7; ++size) {
      if (cluster_fits(info, mp, N, K, size)) {
        candidates.push_back(size);
      }
    }
    int   best    = -1;
    float best_ms = 0.0f;
    for (const int cand : candidates) {
      const float cand_ms =
        time_candidate([&](const uint8_t* w) { return launch_decode(false, A, A_s, w, B_s, C, C_s, mp, N, K, stream, cand); });
      if (rc == LLMMM_OK && cand_ms >= 0.0f && (best < 0 || cand_ms < best_ms)) {
        best    = cand;
        best_ms = cand_ms;
      }
    }
    if (rc == LLMMM_OK && best >= 0) {
      std::lock_guard<std::mutex> lock(g_plan_mutex);
      g_plan_table[{info->device, mp, N, K}] = best;
    }
  }
  cleanup();
  return rc;
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

int llmmm_prepare_workspace(void* device_ptr, size_t bytes, llmmm_stream_t stream)
{
  using namespace llmmm;
  if (device_info() == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  if (device_ptr == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  const int rc = check_workspace_arg(device_ptr, bytes);
  if (rc != LLMMM_OK) {
    return rc;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  LLMMM_CUDA_TRY(cudaMemsetAsync(device_ptr, 0, WS_HEADER_BYTES, s));
  if (bytes > split_workspace_bytes()) {
    LLMMM_CUDA_TRY(cudaMemsetAsync(static_cast<uint8_t*>(device_ptr) + split_workspace_bytes(), 0, bytes - split_workspace_bytes(), s));
  }
  return LLMMM_OK;
}

int llmmm_bind_workspace(void* device_ptr, size_t bytes)
{
  using namespace llmmm;
  const int rc = check_workspace_arg(device_ptr, bytes);
  if (rc != LLMMM_OK) {
    return rc;
  }
  t_ws.ptr   = device_ptr;
  t_ws.bytes = device_ptr ? bytes : 0;
  t_ws_bound = device_ptr != nullptr;
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
    if (check_workspace_arg(device_ptr, bytes) != LLMMM_OK) {
      return LLMMM_ERR_SHAPE;
    }
    // the arrival counters of the pair kernels' split tiles and the flagged words of the decode kernel's partial
    // tiles must start at zero; every launch leaves them at zero again
    LLMMM_CUDA_TRY(cudaMemset(device_ptr, 0, WS_HEADER_BYTES));
    if (bytes > split_workspace_bytes()) {
      LLMMM_CUDA_TRY(cudaMemset(static_cast<uint8_t*>(device_ptr) + split_workspace_bytes(), 0, bytes - split_workspace_bytes()));
    }
    g_scratch_dirty[info->device].store(0);
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
constexpr size_t NOALLOC_BYTES = (size_t)deccfg::MAX_CTAS * 2 * 16 * 128 * sizeof(uint32_t);

// 160 x 2 partial tiles of 16 x 128 self-announcing 32-bit words: 2,621,440 bytes, zero when the library is
// loaded and zero again after every call (a reader clears the words it consumed).
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
  if (const int cluster = planned_cluster(info, M, N, K, nullptr)) {
    // same choice as llmmm_fp8_blockwise_mm_e4m3out makes: the cluster kernel needs no scratch at all
    return launch_decode_cluster_t<16, false>(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K, cluster, info, s);
  }
  // Every call shares the array and leaves its flagged words at zero.  Only after a call whose wait ran out
  // (llmmm_check_status reported it) may set words be left behind: then the array is cleared here first.
  if (g_noalloc_dirty[info->device].exchange(0) != 0) {
    LLMMM_CUDA_TRY(cudaMemsetAsync(scratch, 0, NOALLOC_BYTES, s));
  }
  return launch_decode_t<16, false>(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K,
                                    reinterpret_cast<uint32_t*>(scratch), info, s);
}

