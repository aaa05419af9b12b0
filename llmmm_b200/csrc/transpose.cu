// dst[N,M] = src[M,N]^T for 1-byte and 4-byte elements, M and N multiples of 128 (HBM-bound: every
// byte is read once and written once, both sides in full 128-byte lines).
//
// Replaces the reference's transpose_matrix__aligned_128<T> (src/base/base.cu:9-155), which the FP8
// path uses to turn checkpoint-layout B[K,N] into the K-contiguous B_transposed[N,K] the GEMM reads
// (examples/005.fp8.mm.cu:2657-2660).  The reference transposes 128x128 (1-byte) / 64x64 (4-byte)
// tiles inside one warp's registers; here a CTA stages a tile in shared memory:
//   * 4-byte: 32x32-word tiles, padded rows (33 words);
//   * 1-byte: 128x128-byte tiles; a thread transposes 4x4-byte blocks in registers (byte permutes) so
//     that shared memory is only touched with whole words, stored under an XOR swizzle that keeps both
//     the transposed writes and the row reads free of bank conflicts.
#include "host_common.h"
#include "sm100.cuh"

namespace llmmm {

__global__ void __launch_bounds__(256) transpose_b32_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, int M, int N)
{
  __shared__ uint32_t tile[32][33];
  pdl_launch_dependents();  // see sm100.cuh: the next kernel may start its set-up, this one waits for its predecessor
  pdl_wait();
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;
  const int m0 = blockIdx.y * 32;
  const int n0 = blockIdx.x * 32;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = ty + 8 * j;
    tile[r][tx] = __ldcs(src + (size_t)(m0 + r) * N + n0 + tx);
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = ty + 8 * j;  // output row inside the tile = input column
    __stcs(dst + (size_t)(n0 + r) * M + m0 + tx, tile[tx][r]);
  }
}

__global__ void __launch_bounds__(256) transpose_b8_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int M, int N)
{
  // T[out_row][word]: out_row = input column (0..127), word w holds input rows 4w..4w+3; physical word = w ^ (out_row >> 2)
  __shared__ uint32_t T[128][32];
  pdl_launch_dependents();
  pdl_wait();
  const int tx = threadIdx.x & 31;  // 4-column block of the input tile
  const int ty = threadIdx.x >> 5;
  const int m0 = blockIdx.y * 128;
  const int n0 = blockIdx.x * 128;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int rb = ty + 8 * j;  // 4-row block of the input tile
    uint32_t  r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[i] = __ldcs(reinterpret_cast<const uint32_t*>(src + (size_t)(m0 + 4 * rb + i) * N + n0) + tx);
    }
    // 4x4 byte transpose: t[q] = byte q of r[0..3]
    const uint32_t a0 = __byte_perm(r[0], r[1], 0x5140);  // r0.b0 r1.b0 r0.b1 r1.b1
    const uint32_t a1 = __byte_perm(r[2], r[3], 0x5140);
    const uint32_t a2 = __byte_perm(r[0], r[1], 0x7362);  // r0.b2 r1.b2 r0.b3 r1.b3
    const uint32_t a3 = __byte_perm(r[2], r[3], 0x7362);
    const uint32_t t0 = __byte_perm(a0, a1, 0x5410);
    const uint32_t t1 = __byte_perm(a0, a1, 0x7632);
    const uint32_t t2 = __byte_perm(a2, a3, 0x5410);
    const uint32_t t3 = __byte_perm(a2, a3, 0x7632);
    const int      sw = rb ^ tx;  // rows are 32 words apart, so the bank is the column: distinct over tx
    T[4 * tx + 0][sw] = t0;
    T[4 * tx + 1][sw] = t1;
    T[4 * tx + 2][sw] = t2;
    T[4 * tx + 3][sw] = t3;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int r = ty + 8 * j;  // output row inside the tile
    __stcs(reinterpret_cast<uint32_t*>(dst + (size_t)(n0 + r) * M + m0) + tx, T[r][tx ^ (r >> 2)]);
  }
}

}  // namespace llmmm

extern "C" int llmmm_transpose_aligned_128(void* dst, const void* src, int M, int N, int elem_bytes, llmmm_stream_t stream)
{
  using namespace llmmm;
  if (dst == nullptr || src == nullptr) {
    return set_error(LLMMM_ERR_SHAPE, "null pointer argument");
  }
  if (M < 128 || N < 128 || (M % 128) != 0 || (N % 128) != 0) {
    return set_error(LLMMM_ERR_SHAPE, "M or N can't be divided 128. (got %d %d)", M, N);
  }
  if (elem_bytes != 1 && elem_bytes != 4) {
    return set_error(LLMMM_ERR_UNSUPPORTED, "T is not supported. (element size %d; 1 and 4 bytes are)", elem_bytes);
  }
  if (((uintptr_t)dst | (uintptr_t)src) & 15) {
    return set_error(LLMMM_ERR_SHAPE, "dst and src must be 16-byte aligned");
  }
  if (device_info() == nullptr) {
    return LLMMM_ERR_UNSUPPORTED;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (elem_bytes == 4) {
    LLMMM_CUDA_TRY(launch_pdl(transpose_b32_kernel, dim3(N / 32, M / 32), dim3(256), 0, s, 1, static_cast<uint32_t*>(dst),
                              static_cast<const uint32_t*>(src), M, N));
  }
  else {
    LLMMM_CUDA_TRY(launch_pdl(transpose_b8_kernel, dim3(N / 128, M / 128), dim3(256), 0, s, 1, static_cast<uint8_t*>(dst),
                              static_cast<const uint8_t*>(src), M, N));
  }
  g_launches.fetch_add(1);
  return LLMMM_OK;
}
