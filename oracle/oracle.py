"""numpy/ctypes front end of the CPU oracle (oracle.cpp).  TEST INFRASTRUCTURE.

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import
this module; the product package (llmmm_b200) never does.

Each function names the reference code it restates (paths relative to the
reference project root); the arithmetic itself lives in oracle.cpp.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "liboracle.so"
_lib = None

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i = ctypes.c_int
_i64 = ctypes.c_int64


def build(force: bool = False) -> Path:
    """Compiles liboracle.so with the recipe in oracle/Makefile."""
    if force or not _LIB.exists() or _LIB.stat().st_mtime < (_HERE / "oracle.cpp").stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s", "all"], check=True,
                       capture_output=True)
    return _LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB.exists():
            build()
        L = ctypes.CDLL(str(_LIB))
        L.oracle_num_threads.restype = _i
        L.oracle_set_num_threads.argtypes = [_i]
        L.oracle_e4m3_decode.argtypes = [_u8p, _f32p, _i64]
        L.oracle_e4m3_encode.argtypes = [_f32p, _u8p, _i64]
        L.oracle_f32_to_f16.argtypes = [_f32p, _u16p, _i64]
        L.oracle_f16_to_f32.argtypes = [_u16p, _f32p, _i64]
        L.oracle_f32_to_bf16.argtypes = [_f32p, _u16p, _i64]
        L.oracle_bf16_to_f32.argtypes = [_u16p, _f32p, _i64]
        L.oracle_kahan_gemm.argtypes = [_f32p, _f32p, _f32p, _i, _i, _i, _i, _i]
        L.oracle_double_gemm.argtypes = [_f32p, _f32p, _f32p, _i, _i, _i, _i, _i]
        L.oracle_exact_gemm_f64.argtypes = [_f32p, _f32p, _f64p, _i, _i, _i, _i, _i]
        L.oracle_quant_1x128.argtypes = [_f32p, _u8p, _f32p, _i, _i]
        L.oracle_quant_128x128.argtypes = [_f32p, _u8p, _f32p, _i, _i]
        L.oracle_fp8_blockwise_acc.argtypes = [_u8p, _f32p, _u8p, _f32p, ctypes.c_void_p, ctypes.c_void_p,
                                               _i, _i, _i, _i, _i, _i]
        L.oracle_c_quant_1x128.argtypes = [_f32p, _u8p, _f32p, _i, _i, _i, _i]
        L.oracle_dequant_1x128.argtypes = [_u8p, _f32p, _f32p, _i, _i]
        L.oracle_transpose.argtypes = [ctypes.c_void_p, ctypes.c_void_p, _i, _i, _i]
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


# ------------------------------------------------------------------ codecs --

def e4m3_decode(q: np.ndarray) -> np.ndarray:
    """e4m3 bytes -> float32 (exact)."""
    q = _c(q, np.uint8)
    out = np.empty(q.shape, np.float32)
    lib().oracle_e4m3_decode(q.reshape(-1), out.reshape(-1), q.size)
    return out


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 bytes with `__nv_fp8_e4m3(float)` semantics (RN-even, saturating)."""
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().oracle_e4m3_encode(x.reshape(-1), out.reshape(-1), x.size)
    return out


def to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_f16(x.reshape(-1), out.reshape(-1), x.size)
    return out


def from_f16_bits(b: np.ndarray) -> np.ndarray:
    b = _c(b, np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().oracle_f16_to_f32(b.reshape(-1), out.reshape(-1), b.size)
    return out


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_bf16(x.reshape(-1), out.reshape(-1), x.size)
    return out


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    b = _c(b, np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().oracle_bf16_to_f32(b.reshape(-1), out.reshape(-1), b.size)
    return out


# --------------------------------------------------------- reference GEMMs --

def _rows(M, row0, rows):
    if rows is None:
        row0, rows = 0, M
    assert 0 <= row0 and row0 + rows <= M
    return row0, rows


def kahan_gemm(A: np.ndarray, B: np.ndarray, row0: int = 0, rows: int | None = None) -> np.ndarray:
    """fp32 Kahan-summed GEMM, test/kahan.cu:7-27.  A[M,K], B[K,N] fp32."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    (M, K), N = A.shape, B.shape[1]
    row0, rows = _rows(M, row0, rows)
    C = np.empty((rows, N), np.float32)
    lib().oracle_kahan_gemm(A, B, C, M, N, K, row0, rows)
    return C


def double_gemm(A: np.ndarray, B: np.ndarray, row0: int = 0, rows: int | None = None) -> np.ndarray:
    """fp32 GEMM with a double accumulator, test/kahan.cu:39-56."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    (M, K), N = A.shape, B.shape[1]
    row0, rows = _rows(M, row0, rows)
    C = np.empty((rows, N), np.float32)
    lib().oracle_double_gemm(A, B, C, M, N, K, row0, rows)
    return C


def exact_gemm(A: np.ndarray, B: np.ndarray, row0: int = 0, rows: int | None = None) -> np.ndarray:
    """fp64 accumulation of exact products (ground truth for src/mm/fp16/mm.cuh:85,427)."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    (M, K), N = A.shape, B.shape[1]
    row0, rows = _rows(M, row0, rows)
    C = np.empty((rows, N), np.float64)
    lib().oracle_exact_gemm_f64(A, B, C, M, N, K, row0, rows)
    return C


# -------------------------------------------------------------- quantisers --

def quant_1x128(x: np.ndarray):
    """examples/005.fp8.mm.cu:439-500 <1,128,true>: returns (q[M,K] u8, scale[(K/128),M] f32)."""
    x = _c(x, np.float32)
    M, K = x.shape
    assert K % 128 == 0
    q = np.empty((M, K), np.uint8)
    s = np.empty((K // 128, M), np.float32)
    lib().oracle_quant_1x128(x, q, s, M, K)
    return q, s


def quant_128x128(x: np.ndarray):
    """examples/005.fp8.mm.cu:503-544 <128,128,false>: returns (q u8, scale[(rows/128),(cols/128)])."""
    x = _c(x, np.float32)
    R, C = x.shape
    assert R % 128 == 0 and C % 128 == 0
    q = np.empty((R, C), np.uint8)
    s = np.empty((R // 128, C // 128), np.float32)
    lib().oracle_quant_128x128(x, q, s, R, C)
    return q, s


# ------------------------------------------------------ FP8 blockwise GEMM --

def fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact: bool = False, row0: int = 0, rows: int | None = None):
    """Accumulator of the blockwise GEMM before C is re-quantised
    (examples/005.fp8.mm.cu:1057-1068 and :890-901).
    exact=False: fp32 with the reference's operation order ("T1");
    exact=True: fp64 ground truth for the quantised operands ("T0")."""
    A_q, B_q = _c(A_q, np.uint8), _c(B_q, np.uint8)
    A_s, B_s = _c(A_s, np.float32), _c(B_s, np.float32)
    (M, K), N = A_q.shape, B_q.shape[0]
    assert B_q.shape[1] == K and K % 128 == 0 and N % 128 == 0
    assert A_s.shape == (K // 128, M) and B_s.shape == (N // 128, K // 128)
    row0, rows = _rows(M, row0, rows)
    if exact:
        out = np.empty((rows, N), np.float64)
        lib().oracle_fp8_blockwise_acc(A_q, A_s, B_q, B_s, None, out.ctypes.data, M, N, K, row0, rows, 1)
    else:
        out = np.empty((rows, N), np.float32)
        lib().oracle_fp8_blockwise_acc(A_q, A_s, B_q, B_s, out.ctypes.data, None, M, N, K, row0, rows, 0)
    return out


def c_quant_1x128(acc: np.ndarray):
    """Fused output quantisation, examples/005.fp8.mm.cu:1107-1138:
    returns (C_q[M,N] u8, C_s[(N/128),M] f32)."""
    acc = _c(acc, np.float32)
    M, N = acc.shape
    q = np.empty((M, N), np.uint8)
    s = np.empty((N // 128, M), np.float32)
    lib().oracle_c_quant_1x128(acc, q, s, M, N, M, 0)
    return q, s


def dequant_1x128(q: np.ndarray, s: np.ndarray) -> np.ndarray:
    """float(q[m,n]) * s[n/128, m]  (examples/005.fp8.mm.cu:2865-2869)."""
    q, s = _c(q, np.uint8), _c(s, np.float32)
    M, N = q.shape
    out = np.empty((M, N), np.float32)
    lib().oracle_dequant_1x128(q, s, out, M, N)
    return out


def fp8_blockwise_mm(A_q, A_s, B_q, B_s):
    """Whole fused kernel in the reference's arithmetic: (C_q, C_s, acc_f32)."""
    acc = fp8_blockwise_acc(A_q, A_s, B_q, B_s)
    q, s = c_quant_1x128(acc)
    return q, s, acc


def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float, exact: bool = False) -> np.ndarray:
    """y = x * rsqrt(mean(x^2) + eps) * weight per row.  exact=False: fp32 with the kernel's operation order up to
    the order of the sum of squares (x * inv first, then * weight); exact=True: fp64 ground truth.  The reference
    only plans this hook (README.md:16); the definition is the usual RMSNorm."""
    if exact:
        x64, w64 = x.astype(np.float64), weight.astype(np.float64)
        return x64 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + eps) * w64
    x = _c(x, np.float32)
    ms = ((x.astype(np.float64) ** 2).sum(axis=1, keepdims=True)).astype(np.float32) / np.float32(x.shape[1])
    inv = (np.float32(1) / np.sqrt(ms + np.float32(eps), dtype=np.float32)).astype(np.float32)
    return ((x * inv).astype(np.float32) * _c(weight, np.float32)).astype(np.float32)


def rmsnorm_quant_1x128(x: np.ndarray, weight: np.ndarray, eps: float):
    """RMSNorm followed by the activation quantiser: (q, scale, y_f32, y_f64_truth)."""
    y32 = rmsnorm(x, weight, eps)
    q, s = quant_1x128(y32)
    return q, s, y32, rmsnorm(x, weight, eps, exact=True)


def swiglu(acc: np.ndarray) -> np.ndarray:
    """h[m, i] = silu(acc[m, i]) * acc[m, I + i] for a gate_up accumulator [M, 2I] (gate columns first),
    silu(x) = x / (1 + exp(-x)); computed in the dtype of `acc` (fp32: the kernel's arithmetic up to the
    exponential's last bits; fp64: ground truth).  The reference only plans this fusion (README.md:16), so
    the definition is the usual SwiGLU one."""
    I = acc.shape[1] // 2
    gate, up = acc[:, :I], acc[:, I:]
    one = acc.dtype.type(1)
    with np.errstate(over="ignore"):
        return (gate / (one + np.exp(-gate)) * up).astype(acc.dtype)


def fp8_blockwise_mm_swiglu(A_q, A_s, B_q, B_s, row0: int = 0, rows: int | None = None):
    """gate_up GEMM + SwiGLU + 1x128 quantisation along I: (H_q, H_s, h_f32, h_f64_truth)."""
    h32 = swiglu(fp8_blockwise_acc(A_q, A_s, B_q, B_s, row0=row0, rows=rows))
    h64 = swiglu(fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True, row0=row0, rows=rows))
    q, s = c_quant_1x128(h32)
    return q, s, h32, h64


def qk_norm_rope(acc: np.ndarray, positions, cos, sin, q_weight, k_weight, eps: float, n_q: int, n_kv: int) -> np.ndarray:
    """The qkv hook on an accumulator [M, (n_q + 2 n_kv) * 128], heads of 128 columns (query, key, value):
    query / key heads are RMS-normalised over their 128 values when the weight of their kind is given
    (x * (1 / sqrt(mean(x^2) + eps)) * w) and rotated: y[i] = x[i] cos[p, i] - x[i+64] sin[p, i],
    y[i+64] = x[i+64] cos[p, i] + x[i] sin[p, i], p = positions[m]; value heads pass unchanged.  Computed in the
    dtype of `acc` (fp32: the kernel's arithmetic up to the sum of squares' order and the reciprocal square
    root's last bits; fp64: ground truth).  The reference only plans "norm/rope fusion" (README.md:16); this is
    the usual definition with the half-split pairing."""
    t = acc.dtype.type
    M, N = acc.shape
    x = acc.reshape(M, N // 128, 128).copy()
    c = np.asarray(cos)[np.asarray(positions)].astype(acc.dtype)[:, None, :]  # [M, 1, 64]
    s = np.asarray(sin)[np.asarray(positions)].astype(acc.dtype)[:, None, :]
    for lo, hi, w in ((0, n_q, q_weight), (n_q, n_q + n_kv, k_weight)):
        h = x[:, lo:hi]
        if w is not None:
            ms = (h.astype(np.float64) ** 2).sum(axis=2, keepdims=True).astype(acc.dtype) / t(128)
            inv = (t(1) / np.sqrt(ms + t(eps), dtype=acc.dtype)).astype(acc.dtype)
            h = ((h * inv).astype(acc.dtype) * np.asarray(w).astype(acc.dtype)).astype(acc.dtype)
        x0, x1 = h[..., :64], h[..., 64:]
        x[:, lo:hi] = np.concatenate([x0 * c - x1 * s, x1 * c + x0 * s], axis=2).astype(acc.dtype)
    return x.reshape(M, N)


def fp8_blockwise_mm_qk_norm_rope(A_q, A_s, B_q, B_s, positions, cos, sin, q_weight, k_weight, eps, n_q, n_kv,
                                  row0: int = 0, rows: int | None = None):
    """qkv GEMM + hook + 1x128 quantisation: (C_q, C_s, y_f32, y_f64_truth) for rows [row0, row0 + rows)."""
    n = A_q.shape[0] - row0 if rows is None else rows
    pos = np.asarray(positions)[row0:row0 + n]
    y32 = qk_norm_rope(fp8_blockwise_acc(A_q, A_s, B_q, B_s, row0=row0, rows=rows), pos, cos, sin, q_weight, k_weight,
                       eps, n_q, n_kv)
    y64 = qk_norm_rope(fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True, row0=row0, rows=rows), pos, cos, sin,
                       q_weight, k_weight, eps, n_q, n_kv)
    q, s = c_quant_1x128(y32)
    return q, s, y32, y64


def transpose(x: np.ndarray) -> np.ndarray:
    """src/base/base.cu:125-152 for 1- and 4-byte elements."""
    x = np.ascontiguousarray(x)
    out = np.empty((x.shape[1], x.shape[0]), x.dtype)
    lib().oracle_transpose(x.ctypes.data, out.ctypes.data, x.shape[0], x.shape[1], x.dtype.itemsize)
    return out
