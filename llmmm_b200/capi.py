"""ctypes binding of the C ABI declared in include/llmmm_c.h.

The functions here mirror the reference's host launchers (argument order and
error behaviour): `fp16_mm` is LLMMM::fp16_mm<T> (src/mm/fp16/mm.h:9-10), the
FP8 functions are the launchers of examples/005.fp8.mm.cu:217-246, 547-563 and
2466-2577.  A non-zero status from the library is raised as RuntimeError, the
Python counterpart of the reference's std::runtime_error.

torch is used only to hold device memory and to name the current stream.
There is no fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "libllmmm_b200.so"
_lib = None

_vp = ctypes.c_void_p
_i = ctypes.c_int


def lib() -> ctypes.CDLL:
    """Loads libllmmm_b200.so (built in-tree by llmmm_b200.build)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m llmmm_b200.build`; there is no fallback path")
        L = ctypes.CDLL(str(_LIB_PATH))
        L.llmmm_last_error.restype = ctypes.c_char_p
        L.llmmm_version.restype = ctypes.c_char_p
        L.llmmm_launch_count.restype = ctypes.c_uint64
        L.llmmm_split_launch_count.restype = ctypes.c_uint64
        L.llmmm_fp8_workspace_bytes.restype = ctypes.c_size_t
        L.llmmm_fp8_swiglu_workspace_bytes.restype = ctypes.c_size_t
        L.llmmm_fp8_swiglu_workspace_bytes.argtypes = [_i, _i, _i]
        L.llmmm_fp8_workspace_bytes.argtypes = [_i, _i, _i]
        L.llmmm_set_workspace.argtypes = [_vp, ctypes.c_size_t]
        L.llmmm_check_status.argtypes = [_vp]
        for name in ("llmmm_fp16_mm_f16", "llmmm_fp16_mm_bf16"):
            getattr(L, name).argtypes = [_vp, _vp, _vp, _i, _i, _i, _vp]
        L.llmmm_fp8_blockwise_mm_e4m3out.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
        L.llmmm_fp8_blockwise_mm_e4m3out_noalloc.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
        L.llmmm_fp8_blockwise_mm_swiglu_e4m3out.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
        L.llmmm_fp8_blockwise_mm_qk_norm_rope_e4m3out.argtypes = [_vp] * 9 + [_i, _vp, _vp, ctypes.c_float, _i, _i, _i, _i, _i, _vp]
        L.llmmm_fp8_qk_norm_rope_workspace_bytes.restype = ctypes.c_size_t
        L.llmmm_fp8_qk_norm_rope_workspace_bytes.argtypes = [_i, _i, _i]
        L.llmmm_fp8_blockwise_mm_e4m3out_gather.argtypes = [_vp, _vp, _vp, _vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp),
                                                            _i, _i, _i, _i, _i, _i, _vp]
        L.llmmm_fp8_blockwise_mm_f32out.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
        L.llmmm_fp8_quant_1x128.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
        L.llmmm_fp8_quant_128x128.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
        L.llmmm_fp8_rmsnorm_quant_1x128.argtypes = [_vp, _vp, ctypes.c_float, _vp, _vp, _i, _i, _vp]
        L.llmmm_transpose_aligned_128.argtypes = [_vp, _vp, _i, _i, _i, _vp]
        L.llmmm_selftest_wait_expiry.argtypes = [ctypes.c_uint, _vp]
        L.llmmm_prepare_workspace.argtypes = [_vp, ctypes.c_size_t, _vp]
        L.llmmm_bind_workspace.argtypes = [_vp, ctypes.c_size_t]
        L.llmmm_fp8_blockwise_mm_e4m3out_ws.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, ctypes.c_size_t, _vp]
        L.llmmm_fp8_blockwise_mm_f32out_ws.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, ctypes.c_size_t, _vp]
        for name in ("llmmm_fp16_mm_f16_ws", "llmmm_fp16_mm_bf16_ws"):
            getattr(L, name).argtypes = [_vp, _vp, _vp, _i, _i, _i, _vp, ctypes.c_size_t, _vp]
        _lib = L
    return _lib


EXPORTED_SYMBOLS = (
    "llmmm_last_error", "llmmm_version", "llmmm_fp16_mm_f16", "llmmm_fp16_mm_bf16",
    "llmmm_fp8_blockwise_mm_e4m3out", "llmmm_fp8_blockwise_mm_f32out", "llmmm_fp8_quant_1x128",
    "llmmm_fp8_quant_128x128", "llmmm_fp8_workspace_bytes", "llmmm_set_workspace", "llmmm_check_status",
    "llmmm_launch_count", "llmmm_split_launch_count", "llmmm_set_static_weights", "llmmm_describe_plan", "llmmm_tune",
    "llmmm_fp8_blockwise_mm_e4m3out_noalloc", "llmmm_fp8_blockwise_mm_swiglu_e4m3out",
    "llmmm_fp8_blockwise_mm_e4m3out_gather", "llmmm_fp8_rmsnorm_quant_1x128", "llmmm_fp8_swiglu_workspace_bytes",
    "llmmm_transpose_aligned_128", "llmmm_selftest_wait_expiry",
    "llmmm_fp8_blockwise_mm_qk_norm_rope_e4m3out", "llmmm_fp8_qk_norm_rope_workspace_bytes",
    "llmmm_prepare_workspace", "llmmm_bind_workspace", "llmmm_fp8_blockwise_mm_e4m3out_ws",
    "llmmm_fp8_blockwise_mm_f32out_ws", "llmmm_fp16_mm_f16_ws", "llmmm_fp16_mm_bf16_ws",
)


def _check(status: int) -> None:
    if status != 0:
        raise RuntimeError(f"llmmm status {status}: {lib().llmmm_last_error().decode()}")


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def _dev(t: torch.Tensor, dtype=None) -> int:
    if not t.is_cuda or not t.is_contiguous():
        raise RuntimeError("expected a contiguous CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"expected dtype {dtype}, got {t.dtype}")
    return t.data_ptr()


def launch_count() -> int:
    return int(lib().llmmm_launch_count())


def split_launch_count() -> int:
    """Launches so far that cut the tiles of their last wave along K (needs registered scratch)."""
    return int(lib().llmmm_split_launch_count())


def check_status(stream=None) -> None:
    _check(lib().llmmm_check_status(_stream(stream)))


def fp16_mm(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, M: int, N: int, K: int, stream=None) -> None:
    """C[M,N] = A[M,K] @ B[K,N] for half / bfloat16 (LLMMM::fp16_mm<T>)."""
    if A.dtype == torch.float16:
        fn = lib().llmmm_fp16_mm_f16
    elif A.dtype == torch.bfloat16:
        fn = lib().llmmm_fp16_mm_bf16
    else:
        raise RuntimeError("T is not supported.")
    with torch.cuda.device(A.device):
        _check(fn(_dev(A), _dev(B, A.dtype), _dev(C, A.dtype), M, N, K, _stream(stream)))


def fp8_blockwise_mm(A_q, A_s, B_q, B_s, C_q, C_s, M: int, N: int, K: int, stream=None) -> None:
    """FP8 blockwise GEMM, e4m3 output with fused 1x128 scales
    (fp8_gemm_blockwise_quant_A_1x128__B_128x128__C_1x128__output_fp8*)."""
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_e4m3out(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_q), _dev(B_s, torch.float32), _dev(C_q),
            _dev(C_s, torch.float32), M, N, K, _stream(stream)))


def prepare_workspace(ws: torch.Tensor, stream=None) -> None:
    """Clears the parts of a caller-owned scratch buffer that must be zero between launches (asynchronously)."""
    with torch.cuda.device(ws.device):
        _check(lib().llmmm_prepare_workspace(_dev(ws), ws.numel() * ws.element_size(), _stream(stream)))


def fp8_blockwise_mm_ws(A_q, A_s, B_q, B_s, C_q, C_s, M: int, N: int, K: int, ws, stream=None) -> None:
    """fp8_blockwise_mm with the split-K scratch as an argument (`ws`: a prepared uint8 tensor, or None for no
    scratch); the buffer registered for the device is ignored."""
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_e4m3out_ws(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_q), _dev(B_s, torch.float32), _dev(C_q),
            _dev(C_s, torch.float32), M, N, K, None if ws is None else _dev(ws), 0 if ws is None else ws.numel(),
            _stream(stream)))


def fp8_blockwise_mm_f32_ws(A_q, A_s, B_q, B_s, C, M: int, N: int, K: int, ws, stream=None) -> None:
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_f32out_ws(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_q), _dev(B_s, torch.float32), _dev(C, torch.float32),
            M, N, K, None if ws is None else _dev(ws), 0 if ws is None else ws.numel(), _stream(stream)))


def fp16_mm_ws(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, M: int, N: int, K: int, ws, stream=None) -> None:
    fn = {torch.float16: lib().llmmm_fp16_mm_f16_ws, torch.bfloat16: lib().llmmm_fp16_mm_bf16_ws}.get(A.dtype)
    if fn is None:
        raise RuntimeError("T is not supported.")
    with torch.cuda.device(A.device):
        _check(fn(_dev(A), _dev(B, A.dtype), _dev(C, A.dtype), M, N, K, None if ws is None else _dev(ws),
                  0 if ws is None else ws.numel(), _stream(stream)))


def fp8_blockwise_mm_noalloc(A_q, A_s, B_q, B_s, C_q, C_s, M: int, N: int, K: int, stream=None) -> None:
    """Decode-sized (M <= 16) FP8 blockwise GEMM whose split-K scratch is built into the
    library, for callers that cannot allocate device memory (see include/llmmm_c.h)."""
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_e4m3out_noalloc(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_q), _dev(B_s, torch.float32), _dev(C_q),
            _dev(C_s, torch.float32), M, N, K, _stream(stream)))


def fp8_blockwise_mm_gather(A_q, A_s, B_q, B_s, C_dsts, Cs_dsts, N_total: int, col_offset: int, M: int, N: int, K: int,
                            stream=None) -> None:
    """Column shard [col_offset, col_offset + N) of an N_total-wide product, stored into the full C_q [M, N_total] /
    C_s [N_total/128, M] of every destination (this GPU's and the peers' mapped buffers): the all-gather of an
    N-split happens in the GEMM's epilogue.  Destinations are tensors or raw device addresses."""
    n = len(C_dsts)
    if n != len(Cs_dsts) or not 1 <= n <= 8:
        raise RuntimeError("between 1 and 8 destinations are needed")

    def addr(t, dtype):
        return t if isinstance(t, int) else _dev(t, dtype)

    c_arr = (ctypes.c_void_p * n)(*[addr(t, torch.uint8) for t in C_dsts])
    s_arr = (ctypes.c_void_p * n)(*[addr(t, torch.float32) for t in Cs_dsts])
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_e4m3out_gather(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_q), _dev(B_s, torch.float32), c_arr, s_arr, n, N_total,
            col_offset, M, N, K, _stream(stream)))


def fp8_blockwise_mm_swiglu(A_q, A_s, B_gate_up_q, B_s, H_q, H_s, M: int, I: int, K: int, stream=None) -> None:
    """gate_up projection [2I, K] with the SwiGLU epilogue fused: H = silu(gate) * up, quantised 1x128 along I
    into H_q [M, I] / H_s [I/128, M] (the A operand of the down projection)."""
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_swiglu_e4m3out(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_gate_up_q), _dev(B_s, torch.float32), _dev(H_q),
            _dev(H_s, torch.float32), M, I, K, _stream(stream)))


def fp8_blockwise_mm_qk_norm_rope(A_q, A_s, B_q, B_s, C_q, C_s, positions, cos, sin, q_weight, k_weight, eps: float,
                                  n_q_heads: int, n_kv_heads: int, M: int, N: int, K: int, stream=None) -> None:
    """qkv projection [N, K], N = (n_q_heads + 2 n_kv_heads) * 128, with the per-head RMSNorm of query / key heads
    (weights may be None) and the rotary embedding (pairs (i, i + 64), table row positions[m]) fused in front of
    the 1x128 output quantisation.  cos / sin are [rows, 64]; a position outside [0, rows) is clamped and reported
    by check_status()."""
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != 64:
        raise RuntimeError("cos and sin must both be [rows, 64]")
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_qk_norm_rope_e4m3out(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_q), _dev(B_s, torch.float32), _dev(C_q),
            _dev(C_s, torch.float32), _dev(positions, torch.int32), _dev(cos, torch.float32), _dev(sin, torch.float32),
            int(cos.shape[0]),
            None if q_weight is None else _dev(q_weight, torch.float32),
            None if k_weight is None else _dev(k_weight, torch.float32),
            float(eps), n_q_heads, n_kv_heads, M, N, K, _stream(stream)))


def ensure_qk_norm_rope_workspace(M: int, N: int, K: int, device=None) -> None:
    """Scratch for the decode-sized (M <= 64) form of fp8_blockwise_mm_qk_norm_rope; larger M needs none."""
    ensure_workspace_bytes(int(lib().llmmm_fp8_qk_norm_rope_workspace_bytes(M, N, K)), device)


def fp8_blockwise_mm_f32(A_q, A_s, B_q, B_s, C, M: int, N: int, K: int, stream=None) -> None:
    """FP8 blockwise GEMM, fp32 output
    (fp8_gemm_blockwise_quant_A_1x128__B_128x128__output_fp32)."""
    with torch.cuda.device(A_q.device):
        _check(lib().llmmm_fp8_blockwise_mm_f32out(
            _dev(A_q), _dev(A_s, torch.float32), _dev(B_q), _dev(B_s, torch.float32), _dev(C, torch.float32),
            M, N, K, _stream(stream)))


def fp8_quant_1x128(x, q, scale, M: int, K: int, stream=None) -> None:
    """fp8_blockwise_symmetric_quantization<1,128,true>."""
    with torch.cuda.device(x.device):
        _check(lib().llmmm_fp8_quant_1x128(_dev(x, torch.float32), _dev(q), _dev(scale, torch.float32), M, K,
                                           _stream(stream)))


def fp8_rmsnorm_quant_1x128(x, weight, eps: float, q, scale, M: int, K: int, stream=None) -> None:
    """y = x * rsqrt(mean(x^2) + eps) * weight per row, then the 1x128 quantisation of y (one kernel)."""
    with torch.cuda.device(x.device):
        _check(lib().llmmm_fp8_rmsnorm_quant_1x128(_dev(x, torch.float32), _dev(weight, torch.float32), ctypes.c_float(eps),
                                                   _dev(q), _dev(scale, torch.float32), M, K, _stream(stream)))


def fp8_quant_128x128(x, q, scale, rows: int, cols: int, stream=None) -> None:
    """fp8_blockwise_symmetric_quantization<128,128,false>."""
    with torch.cuda.device(x.device):
        _check(lib().llmmm_fp8_quant_128x128(_dev(x, torch.float32), _dev(q), _dev(scale, torch.float32), rows,
                                             cols, _stream(stream)))


def transpose_aligned_128(dst: torch.Tensor, src: torch.Tensor, M: int, N: int, stream=None) -> None:
    """dst[N,M] = src[M,N]^T for 1- or 4-byte elements (LLMMM::transpose_matrix__aligned_128<T>)."""
    if dst.dtype != src.dtype:
        raise RuntimeError("dst and src must have the same dtype")
    with torch.cuda.device(src.device):
        _check(lib().llmmm_transpose_aligned_128(_dev(dst), _dev(src), M, N, src.element_size(), _stream(stream)))


def fp8_workspace_bytes(M: int, N: int, K: int) -> int:
    return int(lib().llmmm_fp8_workspace_bytes(M, N, K))


_workspaces: dict[int, torch.Tensor] = {}


KINDS = {"fp16": 0, "bf16": 1, "fp8": 2, "fp8_f32out": 3}


def describe_plan(kind: str, M: int, N: int, K: int) -> str:
    """Kernel, tiling, waves and split-K / cluster choice a call with these sizes would get right now."""
    buf = ctypes.create_string_buffer(512)
    _check(lib().llmmm_describe_plan(KINDS[kind], M, N, K, buf, ctypes.c_size_t(len(buf))))
    return buf.value.decode()


def tune(kind: str, N: int, K: int) -> None:
    """One-time per-device set-up of a kernel family (MM_IMPL<T>::tune of the reference's planned functor)."""
    _check(lib().llmmm_tune(KINDS[kind], N, K))


def set_static_weights(enabled: bool) -> None:
    """Promise (or withdraw the promise) that the B operands of later FP8 GEMMs are weights that the kernel
    running just before the GEMM on the same stream never writes; decode-sized calls then prefetch them while
    that kernel is still finishing."""
    _check(lib().llmmm_set_static_weights(1 if enabled else 0))


def clear_workspace() -> None:
    """Unregisters the scratch of the current device (every shape still runs, without split-K)."""
    torch.cuda.synchronize()
    _check(lib().llmmm_set_workspace(None, 0))
    _workspaces.pop(torch.cuda.current_device(), None)


def ensure_swiglu_workspace(M: int, I: int, K: int, device=None) -> None:
    """Scratch for the decode-sized (M <= 64) form of fp8_blockwise_mm_swiglu."""
    ensure_workspace_bytes(int(lib().llmmm_fp8_swiglu_workspace_bytes(M, I, K)), device)


def ensure_workspace(M: int, N: int, K: int, device=None) -> None:
    """Registers a split-K scratch buffer large enough for (M,N,K) on `device`.
    The buffer is owned here (the library never allocates)."""
    ensure_workspace_bytes(fp8_workspace_bytes(M, N, K), device)


def ensure_workspace_bytes(need: int, device=None) -> None:
    """Registers a scratch buffer of at least `need` bytes on `device` (kept if the current one is larger)."""
    if need == 0:
        return
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    cur = _workspaces.get(idx)
    if cur is None or cur.numel() < need:
        cur = torch.zeros(need, dtype=torch.uint8, device=dev)
        _workspaces[idx] = cur
        with torch.cuda.device(dev):
            torch.cuda.synchronize()
            _check(lib().llmmm_set_workspace(cur.data_ptr(), cur.numel()))
