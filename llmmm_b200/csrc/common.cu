// Host-side state behind the C ABI: error text, device info, the device status
// word, TMA descriptor encoding through the driver entry point.
#include <atomic>
#include <cstring>
#include <mutex>

#include <algorithm>
#include <array>
#include <map>

#include "host_common.h"
#include "pair_walk.cuh"
#include "sm100.cuh"

namespace llmmm {

thread_local int t_force_mid = -1;

namespace {
std::map<std::array<int, 3>, int> g_mid_table;
std::mutex                        g_mid_mutex;
}  // namespace

int mid_choice(int device, int N, int K)
{
  std::lock_guard<std::mutex> lock(g_mid_mutex);
  const auto                  it = g_mid_table.find({device, N, K});
  return it == g_mid_table.end() ? -1 : it->second;
}

void record_mid_choice(int device, int N, int K, int choice)
{
  std::lock_guard<std::mutex> lock(g_mid_mutex);
  g_mid_table[{device, N, K}] = choice;
}

std::atomic<int> g_scratch_dirty[64];
std::atomic<int> g_noalloc_dirty[64];

namespace {

thread_local char g_error[512] = "";

// One status word per device that loads the library; written by device-side
// waits that ran out (see mbar_wait), read by llmmm_check_status().
__device__ uint32_t g_status_word;

constexpr int MAX_DEVICES = 64;
DeviceInfo    g_devices[MAX_DEVICES];
bool          g_device_ready[MAX_DEVICES];
std::mutex    g_device_mutex;

using EncodeTiledFn = CUresult (*)(CUtensorMap*,
                                   CUtensorMapDataType,
                                   cuuint32_t,
                                   void*,
                                   const cuuint64_t*,
                                   const cuuint64_t*,
                                   const cuuint32_t*,
                                   const cuuint32_t*,
                                   CUtensorMapInterleave,
                                   CUtensorMapSwizzle,
                                   CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode()
{
  static std::once_flag once;
  std::call_once(once, []() {
    void*                           fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  });
  return g_encode;
}

__global__ void __launch_bounds__(256, 1) pair_probe_kernel() {}

// Number of 2-CTA clusters of a 1-CTA-per-SM kernel that fit on the device at once.
int pair_capacity(int sm_count)
{
  constexpr int smem = 200 * 1024;  // forces one CTA per SM, like the GEMM kernels
  if (cudaFuncSetAttribute(pair_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = dim3(2 * (sm_count / 2));
  cfg.blockDim           = dim3(256);
  cfg.dynamicSmemBytes   = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id               = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs                = attr;
  cfg.numAttrs             = 1;
  int clusters             = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, pair_probe_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters < sm_count / 2 ? clusters : sm_count / 2;
}

}  // namespace

std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_split_launches{0};

int set_error(int code, const char* fmt, ...)
{
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

const DeviceInfo* device_info()
{
  int         dev = -1;
  cudaError_t e   = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    set_error(LLMMM_ERR_UNSUPPORTED, "no usable CUDA device: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (!g_device_ready[dev]) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) {
      set_error(LLMMM_ERR_CUDA, "cudaGetDeviceProperties failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    if (prop.major != 10) {
      set_error(LLMMM_ERR_UNSUPPORTED,
                "device %d is sm_%d%d; this library contains sm_100a code only and has no fallback",
                dev,
                prop.major,
                prop.minor);
      return nullptr;
    }
    void* sp = nullptr;
    e        = cudaGetSymbolAddress(&sp, g_status_word);
    if (e != cudaSuccess) {
      set_error(LLMMM_ERR_CUDA, "cudaGetSymbolAddress(status) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    e = cudaMemset(sp, 0, sizeof(uint32_t));
    if (e != cudaSuccess) {
      set_error(LLMMM_ERR_CUDA, "clearing the status word failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    g_devices[dev].device   = dev;
    g_devices[dev].sm_count = prop.multiProcessorCount;
    // Every kernel here runs one CTA per SM; a pair needs two SMs of one TPC/GPC.  Pairs can be
    // fewer than sm_count / 2 when a GPC has an odd number of usable SMs.
    g_devices[dev].max_pairs = pair_capacity(prop.multiProcessorCount);
    g_devices[dev].status   = static_cast<uint32_t*>(sp);
    g_device_ready[dev]     = true;
  }
  return &g_devices[dev];
}

bool make_tmap_2d(CUtensorMap*        out,
                  const void*         base,
                  CUtensorMapDataType dtype,
                  uint32_t            elem_bytes,
                  uint64_t            inner,
                  uint64_t            outer,
                  uint64_t            row_stride_bytes,
                  uint32_t            box_inner,
                  uint32_t            box_outer,
                  CUtensorMapSwizzle  swizzle)
{
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) {
    set_error(LLMMM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  (void)elem_bytes;
  cuuint64_t dims[2]    = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2]     = {box_inner, box_outer};
  cuuint32_t estr[2]    = {1, 1};
  CUresult   r          = enc(out,
                   dtype,
                   2,
                   const_cast<void*>(base),
                   dims,
                   strides,
                   box,
                   estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(LLMMM_ERR_CUDA,
              "cuTensorMapEncodeTiled failed (%d) for base=%p dims=(%llu,%llu) stride=%llu box=(%u,%u)",
              (int)r,
              base,
              (unsigned long long)inner,
              (unsigned long long)outer,
              (unsigned long long)row_stride_bytes,
              box_inner,
              box_outer);
    return false;
  }
  return true;
}

// Self-test of the bounded wait: one CTA waits on an mbarrier that nothing ever signals, with a short
// limit.  The wait must give up, record its code in the status word and let the kernel end normally.
__device__ uint32_t g_selftest_reached_end;

__global__ void wait_expiry_selftest_kernel(uint32_t* status, unsigned long long limit_ns, uint32_t* reached_end)
{
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_wait_limit(&bar, 0, DEV_WAIT_SELFTEST, &abort_flag, status, limit_ns);
    // a second wait of the same CTA returns at once after the first one gave up
    mbar_wait_limit(&bar, 0, DEV_WAIT_SELFTEST, &abort_flag, status, limit_ns);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *reached_end = 1;
  }
}

SplitPlan plan_split(const DeviceInfo* info, int tiles, int k_steps, int fixed, int per_way_x2, int min_gain, bool count)
{
  const int P = info->max_pairs;
  SplitPlan plan{};
  plan.dp_tiles    = tiles;
  plan.split_s     = 1;
  plan.split_chunk = k_steps;
  plan.pairs       = tiles < P ? tiles : P;
  const Workspace ws         = registered_workspace(info->device);
  const int       tail_tiles = tiles % P;
  if (ws.ptr == nullptr || ws.bytes <= WS_HEADER_BYTES || tail_tiles == 0
      || (size_t)tail_tiles * 16 * sizeof(uint32_t) > WS_SK_COUNTER_BYTES) {
    return plan;
  }
  const long long slots    = (long long)((ws.bytes - WS_HEADER_BYTES) / (SPLIT_SLOT_FLOATS * sizeof(float)));
  // (never beyond SPLIT_MAX_PAIRS slots: the decode kernel's partial words lie behind them and must stay zero)
  const long long avail    = std::min<long long>(std::min<long long>(P, slots), SPLIT_MAX_PAIRS);
  int             max_ways = (int)(avail / tail_tiles);
  max_ways                 = max_ways < SPLIT_MAX_WAYS ? max_ways : SPLIT_MAX_WAYS;
  int ways = 0, chunk = k_steps, best = k_steps - min_gain;
  for (int w = 2; w <= max_ways; ++w) {
    const int c   = (k_steps + w - 1) / w;
    const int est = c + fixed + (per_way_x2 * w) / 2;
    if (est < best) {
      best  = est;
      ways  = (k_steps + c - 1) / c;  // no empty chunks
      chunk = c;
    }
  }
  if (ways >= 2) {
    if (count) {
      g_split_launches.fetch_add(1);
    }
    plan.dp_tiles    = tiles - tail_tiles;
    plan.split_s     = ways;
    plan.split_chunk = chunk;
    plan.split_pairs = tail_tiles * ways;
    plan.pairs       = plan.dp_tiles > 0 ? P : plan.split_pairs;
    plan.counters    = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ws.ptr) + WS_RESERVED_BYTES);
    plan.partials    = reinterpret_cast<float*>(static_cast<uint8_t*>(ws.ptr) + WS_HEADER_BYTES);
  }
  return plan;
}

size_t split_workspace_bytes()
{
  return WS_HEADER_BYTES + (size_t)SPLIT_MAX_PAIRS * SPLIT_SLOT_FLOATS * sizeof(float);
}

}  // namespace llmmm

extern "C" {

int llmmm_selftest_wait_expiry(unsigned int limit_us, llmmm_stream_t stream)
{
  using namespace llmmm;
  const DeviceInfo* info = device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  if (limit_us == 0 || limit_us > 1000000) {
    return set_error(LLMMM_ERR_SHAPE, "limit_us must be in [1, 1000000]");
  }
  uint32_t* reached = nullptr;
  LLMMM_CUDA_TRY(cudaGetSymbolAddress((void**)&reached, g_selftest_reached_end));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  LLMMM_CUDA_TRY(cudaMemsetAsync(reached, 0, sizeof(uint32_t), s));
  wait_expiry_selftest_kernel<<<1, 64, 0, s>>>(info->status, (unsigned long long)limit_us * 1000ull, reached);
  g_launches.fetch_add(1);
  LLMMM_CUDA_TRY(cudaGetLastError());
  LLMMM_CUDA_TRY(cudaStreamSynchronize(s));
  uint32_t done = 0;
  LLMMM_CUDA_TRY(cudaMemcpy(&done, reached, sizeof(done), cudaMemcpyDeviceToHost));
  if (done != 1) {
    return set_error(LLMMM_ERR_CUDA, "the self-test kernel did not reach its end");
  }
  return LLMMM_OK;  // the expiry itself is reported by llmmm_check_status()
}

const char* llmmm_last_error(void)
{
  return llmmm::g_error;
}

const char* llmmm_version(void)
{
  return "llmmm-b200 0.1 (sm_100a)";
}

uint64_t llmmm_split_launch_count(void)
{
  return llmmm::g_split_launches.load();
}

uint64_t llmmm_launch_count(void)
{
  return llmmm::g_launches.load();
}

int llmmm_check_status(llmmm_stream_t stream)
{
  const llmmm::DeviceInfo* info = llmmm::device_info();
  if (info == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  LLMMM_CUDA_TRY(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  uint32_t word = 0;
  LLMMM_CUDA_TRY(cudaMemcpy(&word, info->status, sizeof(word), cudaMemcpyDeviceToHost));
  if (word != 0) {
    cudaMemset(info->status, 0, sizeof(word));
    llmmm::g_scratch_dirty[info->device].store(1);
    llmmm::g_noalloc_dirty[info->device].store(1);
    if (word == llmmm::DEV_BAD_POSITION) {
      return llmmm::set_error(LLMMM_ERR_DEVICE_WAIT, "a row position lay outside the angle tables and was clamped, code 0x%x", word);
    }
    return llmmm::set_error(LLMMM_ERR_DEVICE_WAIT, "a device-side wait ran out, code 0x%x", word);
  }
  return LLMMM_OK;
}

}  // extern "C"
