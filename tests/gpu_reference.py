"""A GPU-side reference for full-matrix checks of the FP8 blockwise GEMM: the double-accumulator GEMM of the
reference's tests (test/kahan.cu:39-56, launch_fp32_naive_mm) restated for the quantised operands and their
per-block scales, i.e. the oracle's ground-truth tier "T0" (oracle.fp8_blockwise_acc(exact=True)):

    acc[m, n] = sum over K-blocks kb of ( sum_{k in kb} a[m, k] * b[n, k] ) * ( A_s[kb, m] * B_s[n / 128, kb] )

with every product and sum in fp64.  It is test infrastructure, written with torch fp64 matmuls (not part of the
product path).  Why that is exact where it matters: e4m3 values are multiples of 2^-9 below 2^9, so a product is a
multiple of 2^-18 below 2^18 and a 128-term block sum needs at most 43 bits: every fp64 partial sum is exact
whatever the order, and the block sum is THE exact sum.  Only the promotion (block sum times scale product,
added over K-blocks) rounds, in fp64, as in the oracle.  tests/test_gpu_full_matrix.py first checks this module
against the CPU oracle on small shapes."""
from __future__ import annotations

import numpy as np
import torch


def e4m3_table(device) -> torch.Tensor:
    """All 256 e4m3 codes as fp64 (the two NaN codes as NaN)."""
    codes = torch.arange(256, dtype=torch.uint8, device=device)
    return codes.view(torch.float8_e4m3fn).to(torch.float64)


def fp8_blockwise_acc_f64(A_q: torch.Tensor, A_s: torch.Tensor, B_q: torch.Tensor, B_s: torch.Tensor,
                          col0: int = 0, cols: int | None = None) -> torch.Tensor:
    """T0 accumulator [M, cols] fp64 for output columns [col0, col0 + cols) (a multiple of 128 each)."""
    M, K = A_q.shape
    N = B_q.shape[0]
    cols = N - col0 if cols is None else cols
    assert col0 % 128 == 0 and cols % 128 == 0 and K % 128 == 0
    lut = e4m3_table(A_q.device)
    acc = torch.zeros(M, cols, dtype=torch.float64, device=A_q.device)
    Bq = B_q[col0:col0 + cols]
    Bs = B_s[col0 // 128:(col0 + cols) // 128].to(torch.float64)
    for kb in range(K // 128):
        a = lut[A_q[:, kb * 128:(kb + 1) * 128].long()]
        b = lut[Bq[:, kb * 128:(kb + 1) * 128].long()]
        p = a @ b.t()
        sc = A_s[kb].to(torch.float64)[:, None] * Bs[:, kb].repeat_interleave(128)[None, :]
        acc += p * sc
    return acc


def e4m3_ulp(codes: torch.Tensor) -> torch.Tensor:
    """Spacing of e4m3 at the magnitude of each code (fp64, in code units)."""
    v = torch.clamp(e4m3_table(codes.device)[codes.long()].abs(), min=2.0 ** -6)
    e = (torch.frexp(v).exponent - 1).clamp(-6, 8)  # floor(log2 v), exactly (a computed log2 may land just below an integer)
    return torch.ldexp(torch.ones_like(v), e - 3)
