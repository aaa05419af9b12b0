// sm_100a device primitives shared by the GEMM kernels: mbarrier waits with a
// time limit, TMA tile copies, TMEM allocation, tcgen05 MMA issue / commit /
// accumulator loads, and the shared-memory / instruction descriptor builders.
//
// These replace the reference's src/util/util.cuh (mma.sync, ldmatrix and
// register-shuffle wrappers, util.cuh:51-235), which has no counterpart on
// the tcgen05 path.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

namespace llmmm {

// Error codes written to the device status word by a wait that ran out.
enum : uint32_t {
  DEV_OK            = 0,
  DEV_WAIT_SMEM_FULL  = 0x101,
  DEV_WAIT_SMEM_EMPTY = 0x102,
  DEV_WAIT_TMEM_FULL  = 0x103,
  DEV_WAIT_TMEM_EMPTY = 0x104,
  DEV_WAIT_SPLITK     = 0x105,
  DEV_WAIT_SELFTEST   = 0x1ff,
  DEV_BAD_POSITION    = 0x201,  // not a wait: a row position outside the angle tables was clamped (qkv hook)
};

// Wall-clock limit of one wait, in nanoseconds of %globaltimer.
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ unsigned long long global_timer_ns()
{
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id()
{
  return threadIdx.x & 31;
}

// Warp-wide changes of the register allowance (warp-specialised kernels hand registers of their control warps
// to the warps that hold accumulators).
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

// Four floats to four e4m3 bytes (round to nearest even, saturate to +-448), first value in the low byte.
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d)
{
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// ------------------------------------------------------------- mbarrier ---

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem()
{
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
  uint32_t ok;
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t"
               "}"
               : "=r"(ok)
               : "r"(smem_u32(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}

// Waits for the phase with the given parity to complete.  The wait is bounded:
// after WAIT_LIMIT_NS it records `code` in the status word and in the CTA's
// abort flag and returns; every later wait of the CTA then returns at once, so
// the kernel always runs to its normal end (where TMEM is released) and the
// host reads the status word instead of a hung context.
__device__ __forceinline__ void mbar_wait_limit(uint64_t*           bar,
                                                uint32_t            parity,
                                                uint32_t            code,
                                                volatile uint32_t*  abort_flag,
                                                uint32_t*           status,
                                                unsigned long long  limit_ns)
{
  if (mbar_try_wait(bar, parity)) {
    return;
  }
  unsigned long long t0    = 0;
  uint32_t           spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) {
        return;
      }
      unsigned long long now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      }
      else if (now - t0 > limit_ns) {
        *abort_flag = code;
        atomicCAS(status, 0u, code);
        return;
      }
    }
  }
}

__device__ __forceinline__ void
mbar_wait(uint64_t* bar, uint32_t parity, uint32_t code, volatile uint32_t* abort_flag, uint32_t* status)
{
  mbar_wait_limit(bar, parity, code, abort_flag, status, WAIT_LIMIT_NS);
}

// ------------------------------------------- programmatic dependent launch ---
//
// A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization may start while its
// predecessor on the stream is still running; pdl_wait() then blocks until that predecessor has
// completed and its memory is visible.  Everything a kernel does before pdl_wait() must touch no global
// memory.  pdl_launch_dependents() lets the NEXT kernel on the stream start its own set-up as soon as
// every CTA of this grid has executed it (or has exited).  Both are no-ops without the attribute.
__device__ __forceinline__ void pdl_launch_dependents()
{
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void pdl_wait()
{
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ------------------------------------------------------------------ TMA ---

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m)
{
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// global -> this CTA's shared memory, completion on an mbarrier of this CTA.
// (The .shared::cluster destination form addressed with a CTA-local shared
// address refers to the issuing CTA; no multicast is used anywhere.)
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y)
{
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               :
               : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void
tma_load_2d_hint(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, uint64_t policy)
{
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
    :
    : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
    : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int x, int y)
{
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit()
{
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template<int N>
__device__ __forceinline__ void tma_store_wait_read()
{
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template<int N>
__device__ __forceinline__ void tma_store_wait_all()
{
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Untiled bulk copies (both addresses 16-byte aligned, size a multiple of 16 bytes).
// shared -> global, completion through the bulk async-group (tma_store_commit / tma_store_wait_all)
__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, uint32_t bytes)
{
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               :
               : "l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}

// global -> this CTA's shared memory, completion on an mbarrier of this CTA (complete_tx of `bytes`)
__device__ __forceinline__ void bulk_load(void* sdst, const void* gsrc, uint32_t bytes, uint64_t* bar)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(smem_u32(sdst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// this CTA's shared memory -> the shared memory of a CTA of the same cluster (both given as 16-byte aligned
// addresses, the destination and its mbarrier as shared::cluster addresses from mapa_shared); the receiver's
// barrier gets complete_tx of `bytes`
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, const void* ssrc, uint32_t bytes, uint32_t bar_cluster_addr)
{
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(dst_cluster_addr), "r"(smem_u32(ssrc)), "r"(bytes), "r"(bar_cluster_addr)
               : "memory");
}

// orders accesses of the generic and the async proxy to any state space (global data handed between them)
__device__ __forceinline__ void fence_proxy_async_all()
{
  asm volatile("fence.proxy.async;" ::: "memory");
}

// L2 eviction policies for TMA loads.
__device__ __forceinline__ uint64_t policy_evict_first()
{
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ uint64_t policy_evict_last()
{
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ----------------------------------------------------------------- TMEM ---

// Executed by one full warp.  Writes the TMEM base address to *dst (shared).
template<uint32_t COLS>
__device__ __forceinline__ void tmem_alloc(uint32_t* dst)
{
  static_assert(COLS >= 32 && COLS <= 512 && (COLS & (COLS - 1)) == 0, "TMEM columns: power of two in [32,512]");
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "n"(COLS)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

template<uint32_t COLS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr)
{
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(COLS) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Makes the mbarrier track completion of all tcgen05.mma issued so far by
// this thread (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], issued by one thread.
__device__ __forceinline__ void
tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "}"
               :
               : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

__device__ __forceinline__ void
tc_mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
               "}"
               :
               : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

// Each lane of the warp reads 32 consecutive fp32 columns of its own TMEM lane
// (lane quarter = warp index within its warpgroup).  Asynchronous until
// tmem_ld_wait().
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
                 "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                 "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------- descriptors ---

// 64-bit shared-memory matrix descriptor of tcgen05.mma for a 128-byte
// swizzled tile.  Fields: start address >> 4 (bits 0-13), leading-dimension
// byte offset >> 4 (16-29), stride-dimension byte offset >> 4 (32-45),
// descriptor version 1 (46-47), swizzle mode 2 = 128 B (61-63).
//  K-major operand (rows of 128 B along K): sbo = 1024 (8 rows), lbo unused.
//  MN-major operand (rows of 128 B along M/N, one row per k): sbo = 1024
//   (8 k), lbo = bytes between successive 64-element groups along M/N.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// 32-bit instruction descriptor for kind::f16 / kind::f8f6f4 with an fp32
// accumulator.  Fields: D format (bits 4-5: 1 = f32), A format (7-9),
// B format (10-12), A major (15), B major (16) with 0 = K-major and
// 1 = MN-major, N >> 3 (17-22), M >> 4 (24-28).
// Formats: kind::f16 0 = f16, 1 = bf16; kind::f8f6f4 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t
make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major, uint32_t b_mn_major, uint32_t m, uint32_t n)
{
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17)
         | ((m >> 4) << 24);
}

// ------------------------------------------------- CTA pairs (cluster of 2) --
//
// With tcgen05.mma.cta_group::2 one thread of the even ("leader") CTA of a pair
// issues an MMA of M = 256: each CTA's tensor core computes its own 128 rows
// from its own shared memory A tile, and each CTA supplies half of the N
// columns of B.  No TMA multicast is involved: every CTA loads exactly the
// bytes it owns; only mbarrier signals cross the pair.

__device__ __forceinline__ uint32_t cluster_ctarank()
{
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t smem_addr, uint32_t rank)
{
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Arrival without release semantics: for hand-offs whose ordering is already given by
// tcgen05.wait::ld + tcgen05.fence::before_thread_sync ("I have finished reading TMEM").  A
// cluster-scope release would wait for every outstanding memory operation of the thread.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr)
{
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void cluster_sync_all()
{
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The two halves of cluster_sync_all(), for work that can go between them.
__device__ __forceinline__ void cluster_arrive()
{
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait()
{
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// TMA tile load into this CTA's shared memory whose completion is signalled on
// an mbarrier given by shared::cluster address (this CTA's or its pair's).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y)
{
  asm volatile(
    "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
    :
    : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_cluster_addr)
    : "memory");
}

// Completion of all MMAs issued so far by this thread arrives on the mbarrier
// at the same shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar)
{
  const uint16_t mask = 3;
  asm volatile(
    "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
      smem_u32(bar)),
    "h"(mask)
    : "memory");
}

__device__ __forceinline__ void
tc_mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "}"
               :
               : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

__device__ __forceinline__ void
tc_mma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
               "}"
               :
               : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

}  // namespace llmmm
