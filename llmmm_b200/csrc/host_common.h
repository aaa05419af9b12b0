// Host-side helpers shared by the launchers behind the C ABI: error text,
// per-device state (SM count, device status word), TMA descriptor encoding.
#pragma once

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/llmmm_c.h"

namespace llmmm {

// Kernels launched by this library in this process (llmmm_launch_count()).
extern std::atomic<uint64_t> g_launches;
// ... and how many of them cut the tiles of their last wave along K (llmmm_split_launch_count()).
extern std::atomic<uint64_t> g_split_launches;

// Records a message for llmmm_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...);

struct DeviceInfo {
  int       device;
  int       sm_count;
  int       max_pairs;  // CTA pairs (clusters of 2, one CTA per SM) that can be resident at once
  uint32_t* status;     // device address of the status word of this device
};

// Info for the current device; queried once per device.  Returns nullptr (and
// sets the error text) when the device is not an sm_100 part or a CUDA call
// fails.
const DeviceInfo* device_info();

// Encodes a 2-D tiled TMA descriptor.  `inner` is the contiguous dimension.
// Returns false (error text set) when the driver refuses the arguments.
bool make_tmap_2d(CUtensorMap*        out,
                  const void*         base,
                  CUtensorMapDataType dtype,
                  uint32_t            elem_bytes,
                  uint64_t            inner,
                  uint64_t            outer,
                  uint64_t            row_stride_bytes,
                  uint32_t            box_inner,
                  uint32_t            box_outer,
                  CUtensorMapSwizzle  swizzle);

// Decode-sized (M <= 64) split-K FP8 path (fp8_decode.cu).  Returns -1 when it
// does not apply, otherwise an LLMMM_* status.  force_cluster >= 0 overrides the planned choice
// (0: stream-K through the registered scratch, 2..7: clusters of that size); the tuner uses it.
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
                  int          force_cluster = -1);
// Times the candidate plans of the decode kernel for an [N, K] weight at M = 16, 32 and 64 on the current device
// and records the winners (llmmm_tune).  Allocates and frees temporary operands.
int tune_decode(const DeviceInfo* info, int N, int K);

// FP8 GEMMs of 65..128 rows run on the single-CTA kernel (128-row tiles) or on the pair kernel (256-row tiles, half
// empty, but its last wave can be cut along K).  llmmm_tune measures both for a weight shape and records the
// winner; `mid_choice` returns it (-1: not measured, 0: single-CTA kernel, 1: pair kernel).  `t_force_mid` >= 0
// overrides everything for the calling thread (the tuner's own launches).
int  mid_choice(int device, int N, int K);
void record_mid_choice(int device, int N, int K, int choice);
extern thread_local int t_force_mid;
// Launcher of the general FP8 kernels (fp8_mm.cu), e4m3 output; used by the tuner.
int launch_fp8_e4m3(const void* A, const float* A_s, const void* B, const float* B_s, void* C, float* C_s, int M, int N, int K,
                    cudaStream_t stream);

// Set by llmmm_check_status() when it reports a device-side wait that ran out: the decode kernel's flagged
// partial words (registered scratch / built-in scratch) may then hold leftovers and are cleared before the next use.
extern std::atomic<int> g_scratch_dirty[64];
extern std::atomic<int> g_noalloc_dirty[64];

// Caller-owned scratch registered with llmmm_set_workspace() for a device.  Layout: 16 KB unused, arrival
// counters of the split tiles of the pair kernels (zero between launches), the pair kernels' partial tiles
// (up to split_workspace_bytes()), then the decode kernel's flagged partial words (zero between launches).
constexpr size_t WS_RESERVED_BYTES = 16384;  // unused (kept so that the layout behind it does not move)
constexpr size_t WS_SK_COUNTER_BYTES     = 16384;
constexpr size_t WS_HEADER_BYTES         = WS_RESERVED_BYTES + WS_SK_COUNTER_BYTES;

struct Workspace {
  void*  ptr   = nullptr;
  size_t bytes = 0;
};
// The scratch a launch on the calling thread may use: the buffer bound to this thread (explicit-workspace entry
// points, llmmm_bind_workspace) if there is one, else the one registered for the device.
Workspace registered_workspace(int device);
// True while the calling thread has its own scratch bound (its owner keeps it clean; the per-device "dirty" mark
// of the registered buffer does not apply to it).
bool thread_workspace_bound();

// Binds a scratch buffer to the calling thread for the lifetime of the object (nullptr: "no scratch").
class ScopedWorkspace {
public:
  ScopedWorkspace(void* ptr, size_t bytes);
  ~ScopedWorkspace();
  ScopedWorkspace(const ScopedWorkspace&)            = delete;
  ScopedWorkspace& operator=(const ScopedWorkspace&) = delete;

private:
  Workspace prev_;
  bool      prev_bound_;
};
// 256-byte aligned and at least the header, or null with zero bytes; sets the error text otherwise.
int check_workspace_arg(const void* ptr, size_t bytes);

// Scratch the pair kernels want for splitting the tiles of their last wave (pair_walk.cuh).
size_t split_workspace_bytes();
// Scratch of the decode kernel for M rows (header + partial tiles), fp8_decode.cu.
size_t decode_workspace_bytes(int M);
// SwiGLU + 1x128 quantisation of a gate_up accumulator acc [M, 2I] fp32 (quant.cu): the second step of the
// decode-sized form of llmmm_fp8_blockwise_mm_swiglu_e4m3out.
int launch_swiglu_quant(const float* acc, void* H, float* H_s, int M, int I, cudaStream_t stream);

// What the qkv projection's epilogue hook needs: heads of 128 columns, first n_q query heads, then n_kv key heads,
// the rest value heads.  Query and key heads are RMS-normalised over their 128 values (weights q_w / k_w; a null
// pointer skips the normalisation for that kind) and rotated (pairs (i, i + 64), angle table row pos[m]); value
// heads pass unchanged.
struct RopeHook {
  const float* cos;  // [positions, 64]
  const float* sin;  // [positions, 64]
  const int*   pos;  // [M]
  const float* q_w;  // [128] or null
  const float* k_w;  // [128] or null
  float        eps;
  int          n_q;
  int          n_kv;
  int          rows;  // rows of the angle tables: a position outside [0, rows) is clamped and reported in the status word
};
int launch_rope_quant(const float* acc, void* C, float* C_s, const RopeHook& hook, int M, int N, uint32_t* status, cudaStream_t stream);

// What the launch heuristics choose for a problem, as text (llmmm_describe_plan), and the one-time set-up of
// every kernel of a family on the current device (llmmm_tune): function attributes, occupancy queries.
void describe_fp16_plan(const DeviceInfo* info, bool bf16, int M, int N, int K, char* buf, size_t len);
void describe_fp8_plan(const DeviceInfo* info, bool out_f32, int M, int N, int K, char* buf, size_t len);
bool describe_decode_plan(const DeviceInfo* info, int M, int N, int K, char* buf, size_t len);  // false: not a decode shape
int  warm_fp16_kernels(const DeviceInfo* info);
int  warm_fp8_kernels(const DeviceInfo* info);
int  warm_decode_kernels(const DeviceInfo* info);

// Launches `kernel` with programmatic stream serialisation allowed (the kernel must execute pdl_wait()
// before its first access to global memory, see sm100.cuh) and, if cluster > 1, as clusters of that size.
template<typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster,
                       Args&&... args)
{
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = grid;
  cfg.blockDim           = block;
  cfg.dynamicSmemBytes   = smem;
  cfg.stream             = stream;
  cudaLaunchAttribute attr[2];
  unsigned            n                              = 0;
  attr[n].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = 1;
  ++n;
  if (cluster > 1) {
    attr[n].id               = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs    = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define LLMMM_CUDA_TRY(call)                                                                                           \
  do {                                                                                                                 \
    cudaError_t e__ = (call);                                                                                          \
    if (e__ != cudaSuccess) {                                                                                          \
      return ::llmmm::set_error(LLMMM_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__));                      \
    }                                                                                                                  \
  } while (0)

}  // namespace llmmm
