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
constexpr int      STAGES        = 8;
constexpr int      THREADS       = 192;
constexpr uint32_t W_BYTES       = 128 * BK;
constexpr int      MAX_CTAS      = 256;
constexpr int      MAX_GROUPS    = 4096;                 // counters: N <= 524288
constexpr size_t   COUNTER_BYTES = MAX_GROUPS * sizeof(uint32_t);
constexpr uint32_t TMEM_COLS     = 128;  // two partial stages of up to 64 columns
}  // namespace deccfg

template<int MP>
struct DecodeSmem {
  static constexpr uint32_t X_BYTES    = MP * deccfg::BK;
  static constexpr uint32_t OFF_W      = 0;
  static constexpr uint32_t OFF_X      = deccfg::STAGES * deccfg::W_BYTES;
  static constexpr uint32_t OFF_BAR    = OFF_X + deccfg::STAGES * X_BYTES;
  static constexpr uint32_t SMEM_BYTES = OFF_BAR + 2048 + 1024;
};

struct DecodeBars {
  uint64_t full[deccfg::STAGES];
  uint64_t empty[deccfg::STAGES];
  uint64_t part_full[2];
  uint64_t part_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t last_flag;
  uint32_t pad;
  float    amax[4][64];
};

__device__ __forceinline__ void epilogue_bar_sync()
{
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// unit u of the (group, K-block) grid belongs to CTA ((u+1)*G - 1) / U, the
// largest c with floor(c*U/G) <= u.
__device__ __forceinline__ int cta_of_unit(long long u, int G, long long U)
{
  return (int)(((u + 1) * G - 1) / U);
}

template<int MP, bool OUT_F32>
__global__ void __launch_bounds__(deccfg::THREADS, 1) fp8_decode_kernel(const __grid_constant__ CUtensorMap tm_w,
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

  const int       KB      = K / BK;
  const long long U       = (long long)(N / 128) * KB;
  const int       G       = gridDim.x;
  const long long u_begin = ((long long)blockIdx.x * U) / G;
  const long long u_end   = ((long long)(blockIdx.x + 1) * U) / G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int p = 0; p < 2; ++p) {
      mbar_init(&bars->part_full[p], 1);
      mbar_init(&bars->part_empty[p], 4);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc<TMEM_COLS>(&bars->tmem_base);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();  // weights are read once
      const uint64_t pol_x = policy_evict_last();   // activations are re-read by every CTA
      uint32_t       it    = 0;
      for (long long u = u_begin; u < u_end; ++u, ++it) {
        const int      nb = (int)(u / KB);
        const int      kb = (int)(u % KB);
        const uint32_t s  = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        mbar_wait(&bars->empty[s], ph ^ 1, DEV_WAIT_SMEM_EMPTY, abort_flag, status);
        mbar_arrive_expect_tx(&bars->full[s], W_BYTES + L::X_BYTES);
        tma_load_2d_hint(smem + L::OFF_W + s * W_BYTES, &tm_w, &bars->full[s], kb * BK, nb * 128, pol_w);
        tma_load_2d_hint(smem + L::OFF_X + s * L::X_BYTES, &tm_x, &bars->full[s], kb * BK, 0, pol_x);
      }
    }
  }
  else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*e4m3*/ 0, 0, 0, 0, 128, MP);
      uint32_t           it    = 0;
      for (long long u = u_begin; u < u_end; ++u, ++it) {
        const uint32_t s  = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        const uint32_t p  = it & 1;
        const uint32_t pp = (it >> 1) & 1;
        mbar_wait(&bars->part_empty[p], pp ^ 1, DEV_WAIT_TMEM_EMPTY, abort_flag, status);
        mbar_wait(&bars->full[s], ph, DEV_WAIT_SMEM_FULL, abort_flag, status);
        tc_fence_after_sync();
        const uint64_t dw = make_smem_desc_sw128(smem_u32(smem + L::OFF_W + s * W_BYTES), 0, 1024);
        const uint64_t dx = make_smem_desc_sw128(smem_u32(smem + L::OFF_X + s * L::X_BYTES), 0, 1024);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          tc_mma_f8(tmem_base + p * 64, dw + (uint64_t)((kk * UMMA_K) >> 4), dx + (uint64_t)((kk * UMMA_K) >> 4), idesc, kk != 0);
        }
        tc_commit(&bars->empty[s]);
        tc_commit(&bars->part_full[p]);
      }
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

    long long u = u_begin;
    while (u < u_end) {
      const int       nb    = (int)(u / KB);
      const int       kb0   = (int)(u % KB);
      const long long left  = u_end - u;
      const int       kb1   = (left < (long long)(KB - kb0)) ? kb0 + (int)left : KB;
      const bool      whole = (kb0 == 0 && kb1 == KB);

      float acc[MP];
#pragma unroll
      for (int i = 0; i < MP; ++i) {
        acc[i] = 0.0f;
      }
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const uint32_t p  = it & 1;
        const uint32_t pp = (it >> 1) & 1;
        const float    b  = __ldg(B_s + (size_t)nb * KB + kb);
        const float*   as = A_s + (size_t)kb * M;
        mbar_wait(&bars->part_full[p], pp, DEV_WAIT_TMEM_FULL, abort_flag, status);
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < MP / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x32b_x16(tmem_base + p * 64 + t_lane + c * 16, v);
          tmem_ld_wait();
          if (c == MP / 16 - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(&bars->part_empty[p]);
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int   m  = c * 16 + i;
            const float a  = (m < M) ? __ldg(as + m) : 0.0f;
            const float sc = __fmul_rn(a, b);  // one fp32 rounding of the scale product
            acc[m]         = __fmaf_rn(__uint_as_float(v[i]), sc, acc[m]);
          }
        }
      }
      u += (kb1 - kb0);

      bool finish = whole;
      if (!whole) {
        // publish this CTA's partial, then see whether it was the last to arrive
        const int slot = blockIdx.x * 2 + (kb0 == 0 ? 1 : 0);  // run begins inside the group -> slot 0
        float*    dst  = partials + (size_t)slot * (MP * 128);
#pragma unroll
        for (int i = 0; i < MP; ++i) {
          __stcg(dst + i * 128 + n_local, acc[i]);
        }
        __threadfence();
        epilogue_bar_sync();
        const int c_lo = cta_of_unit((long long)nb * KB, G, U);
        const int c_hi = cta_of_unit((long long)(nb + 1) * KB - 1, G, U);
        if (et == 0) {
          const uint32_t old = atomicAdd(&counters[nb], 1u);
          const bool     lst = (old == (uint32_t)(c_hi - c_lo));
          if (lst) {
            counters[nb] = 0;  // ready for the next launch
          }
          bars->last_flag = lst ? 1u : 0u;
        }
        epilogue_bar_sync();
        finish = bars->last_flag != 0;
        if (finish) {
          __threadfence();
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            acc[i] = 0.0f;
          }
          for (int c = c_lo; c <= c_hi; ++c) {
            // CTA c's run begins inside this group (slot 0) unless it began earlier (slot 1)
            const long long cs  = ((long long)c * U) / G;
            const int       sl  = c * 2 + ((cs / KB) == nb && (cs % KB) != 0 ? 0 : 1);
            const float*    src = partials + (size_t)sl * (MP * 128);
#pragma unroll
            for (int i = 0; i < MP; ++i) {
              acc[i] += __ldcg(src + i * 128 + n_local);
            }
          }
        }
        epilogue_bar_sync();  // last_flag may be rewritten by the next segment
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
          // group absmax over the 128 lanes: shuffles inside a warp, then 4 warps through shared memory
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            float a = fabsf(acc[i]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            }
            if (lane == 0) {
              bars->amax[ew][i] = a;
            }
          }
          epilogue_bar_sync();
          uint8_t* C = reinterpret_cast<uint8_t*>(C_out);
#pragma unroll
          for (int i = 0; i < MP; ++i) {
            if (i < M) {
              const float amax = fmaxf(fmaxf(bars->amax[0][i], bars->amax[1][i]), fmaxf(bars->amax[2][i], bars->amax[3][i]));
              const float inv  = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 0.0f;
              C[(size_t)i * N + n_glob] = (uint8_t)__nv_cvt_float_to_fp8(acc[i] * inv, __NV_SATFINITE, __NV_E4M3);
              if (et == i) {
                C_s[(size_t)nb * M + i] = __fdiv_rn(amax, 448.0f);
              }
            }
          }
          epilogue_bar_sync();  // bars->amax is reused by the next segment
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

// ------------------------------------------------------------ host side ---

namespace {
struct Workspace {
  void*  ptr   = nullptr;
  size_t bytes = 0;
};
Workspace  g_ws[64];
std::mutex g_ws_mutex;

int padded_m(int M)
{
  return M <= 16 ? 16 : (M <= 32 ? 32 : 64);
}
}  // namespace

size_t decode_workspace_bytes(int M)
{
  return deccfg::COUNTER_BYTES + (size_t)deccfg::MAX_CTAS * 2 * padded_m(M) * 128 * sizeof(float);
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
                           void*             ws,
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
      fp8_decode_kernel<MP, OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM_BYTES));
    attr_set[info->device] = true;
  }
  const long long U = (long long)(N / 128) * (K / BK);
  int             G = info->sm_count < MAX_CTAS ? info->sm_count : MAX_CTAS;
  if ((long long)G > U) {
    G = (int)U;
  }
  uint32_t* counters = static_cast<uint32_t*>(ws);
  float*    partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + COUNTER_BYTES);
  fp8_decode_kernel<MP, OUT_F32><<<G, THREADS, L::SMEM_BYTES, stream>>>(
    tm_w, tm_x, A_s, B_s, C, C_s, M, N, K, partials, counters, info->status);
  g_launches.fetch_add(1);
  LLMMM_CUDA_TRY(cudaGetLastError());
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
  if (M > 64 || N / 128 > deccfg::MAX_GROUPS) {
    return -1;
  }
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  Workspace ws;
  {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    ws = g_ws[info->device];
  }
  if (ws.ptr == nullptr || ws.bytes < decode_workspace_bytes(M)) {
    return -1;
  }
  const int mp = padded_m(M);
#define LLMMM_DECODE_CASE(MPV)                                                                                         \
  if (mp == MPV) {                                                                                                     \
    return out_f32 ? launch_decode_t<MPV, true>(A, A_s, B, B_s, C, C_s, M, N, K, ws.ptr, info, stream) :               \
                     launch_decode_t<MPV, false>(A, A_s, B, B_s, C, C_s, M, N, K, ws.ptr, info, stream);               \
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
  if (M < 1 || M > 64 || N / 128 > llmmm::deccfg::MAX_GROUPS) {
    return 0;
  }
  return llmmm::decode_workspace_bytes(M);
}

int llmmm_set_workspace(void* device_ptr, size_t bytes)
{
  using namespace llmmm;
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  if (device_ptr != nullptr) {
    if (((uintptr_t)device_ptr & 255) != 0 || bytes < deccfg::COUNTER_BYTES) {
      return set_error(LLMMM_ERR_SHAPE, "workspace must be 256-byte aligned and at least %zu bytes", deccfg::COUNTER_BYTES);
    }
    // the arrival counters must start at zero; every launch leaves them at zero again
    LLMMM_CUDA_TRY(cudaMemset(device_ptr, 0, deccfg::COUNTER_BYTES));
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
  if (M < 1 || M > NOALLOC_MAX_M || N / 128 > deccfg::MAX_GROUPS) {
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
  // The array keeps whatever the previous call left.  Partial tiles are always
  // written before they are read, but the arrival counters of the groups this
  // call uses must start at zero.
  LLMMM_CUDA_TRY(cudaMemsetAsync(scratch, 0, (size_t)(N / 128) * sizeof(uint32_t), s));
  return launch_decode_t<16, false>(A, A_scale_t, B_t, B_scale_t, C, C_scale_t, M, N, K, scratch, info, s);
}

