"""B200 (sm_100a) GEMM library for the LLMMM hot path: FP16/BF16 GEMM and FP8
e4m3 blockwise-quantised GEMM with fused 1x128 output quantisation.

The compute lives in libllmmm_b200.so (hand-written CUDA behind the C ABI of
include/llmmm_c.h); this package is the Python plumbing around it: the ctypes
binding (`capi`), the multi-GPU partitioning helpers (`shard`) and the in-tree
build (`build`).
"""
from . import capi, shard  # noqa: F401

__all__ = ["capi", "shard"]
