// Drop-in for the part of the reference's src/base/base.h that the hot path uses:
// LLMMM::transpose_matrix__aligned_128<T> (src/base/base.h:8-9), forwarded to the C ABI.  The
// mma.sync fragment pre-swizzles declared next to it in the reference (construct_m16n8k32_*_layout)
// have no counterpart: tcgen05 reads operands from shared memory through descriptors.
#pragma once

#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

#include "llmmm_c.h"

namespace LLMMM {

template<typename T>
void transpose_matrix__aligned_128(T* dst, T* src, int M, int N, cudaStream_t stream)
{
  static_assert(sizeof(T) == 1 || sizeof(T) == 4, "1-byte and 4-byte elements, as in the reference");
  if (llmmm_transpose_aligned_128(dst, src, M, N, (int)sizeof(T), stream) != LLMMM_OK) {
    throw std::runtime_error(std::string(llmmm_last_error()));
  }
}

}  // namespace LLMMM
