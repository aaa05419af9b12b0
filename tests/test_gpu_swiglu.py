"""gate_up GEMM with the SwiGLU epilogue fused, against the oracle.

This is a floating-point epilogue (an exponential and a division per element), so the gate is a tolerance,
stated here: the fp32 h the kernel quantises may differ from the fp64 truth by 2e-5 of the row's largest |h|
(GEMM accumulation noise 4e-6 as for the plain kernel, amplified by silu' <= 1.1 and the product with `up`, plus
the fast exponential / division, about 2^-21 relative).  On the outputs that means: scales within 2e-5 relative
of the oracle's, de-quantised values within the oracle's own error + 1 e4m3 ulp * scale + that bound, bytes
overwhelmingly identical, and the consumer property: feeding (H_q, H_s) to the down projection gives what
feeding the oracle's (H_q, H_s) gives, within the same bound.

Budget of the approximate intrinsics in the epilogue (CUDA's documented maximum errors): `__expf(x)` is
2 + floor(|1.173 x|) ulp -- where silu's value matters (|g| <= 16, beyond that exp(-g) is below 2^-23 of 1 or the
result below 2^-23 of the row maximum) at most 20 ulp = 2.4e-6 relative of exp(-g), which enters h through
1 / (1 + exp(-g)) with a weight <= 1; `__fdividef` is 2 ulp = 2.4e-7.  Together <= 2.7e-6 relative of h, well inside
the 2e-5 gate, whose larger part is the accumulation noise of the GEMM."""
import numpy as np
import pytest
import torch

from helpers import e4m3_ulp, fp8_sources
from test_gpu_fp8 import to_dev

pytestmark = pytest.mark.gpu


def make_case(oracle, seed, M, I, K):
    x, w = fp8_sources(seed, M, 2 * I, K, w_std=0.05)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    return A_q, A_s, B_q, B_s


def run(capi, cuda, case, M, I, K, launches=1):
    dA, dAs, dB, dBs = to_dev(cuda, *case)
    Hq = torch.full((M, I), 0xAA, dtype=torch.uint8, device=cuda)
    Hs = torch.full((I // 128, M), float("nan"), device=cuda)
    before = capi.launch_count()
    capi.fp8_blockwise_mm_swiglu(dA, dAs, dB, dBs, Hq, Hs, M, I, K)
    torch.cuda.synchronize()
    capi.check_status()
    assert capi.launch_count() == before + launches
    return Hq.cpu().numpy(), Hs.cpu().numpy()


def check(oracle, case, gq, gs, rows=None):
    M = gq.shape[0]
    r0, n = (0, M) if rows is None else rows
    oq, os_, h32, h64 = oracle.fp8_blockwise_mm_swiglu(*case, row0=r0, rows=n)
    gq, gs = gq[r0:r0 + n], gs[:, r0:r0 + n]
    assert np.isfinite(gs).all()
    row_amax = np.abs(h64).max(axis=1, keepdims=True) + 1e-30
    ok = os_ > 0
    assert (np.abs(gs[ok] / os_[ok] - 1) <= 2e-5).all(), float(np.abs(gs[ok] / os_[ok] - 1).max())
    assert (gs[~ok] == 0).all()
    scale_e = np.repeat(gs.T, 128, axis=1).astype(np.float64)
    deq = oracle.e4m3_decode(gq) * scale_e
    o_deq = oracle.e4m3_decode(oq) * np.repeat(os_.T, 128, axis=1).astype(np.float64)
    ulp = e4m3_ulp(oracle.e4m3_decode(gq)) * scale_e
    assert (np.abs(deq - h64) <= np.abs(o_deq - h64) + ulp + 2e-5 * row_amax).all()
    assert (gq == oq).mean() > 0.99


@pytest.mark.parametrize("shape", [(256, 128, 128), (256, 512, 1024), (200, 384, 256), (1, 256, 512), (640, 1152, 384)])
def test_swiglu_small_shapes(capi, oracle, cuda, shape):
    M, I, K = shape
    case = make_case(oracle, 90, M, I, K)
    capi.clear_workspace()  # the fused 256-row kernel for every M (with scratch, M <= 64 takes the two-kernel path)
    gq, gs = run(capi, cuda, case, M, I, K)
    check(oracle, case, gq, gs)


def test_swiglu_qwen3_4b_prefill_and_down_projection(capi, oracle, cuda):
    # Qwen3-4B MLP at M = 1024: gate_up [2*9728, 2560] fused, then the down projection [2560, 9728] consumes H
    M, I, K = 1024, 9728, 2560
    case = make_case(oracle, 91, M, I, K)
    gq, gs = run(capi, cuda, case, M, I, K)
    check(oracle, case, gq, gs, rows=(M - 8, 8))
    check(oracle, case, gq, gs, rows=(300, 4))
    # all-zero activations rows: zero bytes and zero scales (the defined all-zero case), other rows untouched
    A_q0 = case[0].copy()
    A_q0[100:164] = 0
    zq, zs = run(capi, cuda, (A_q0, *case[1:]), M, I, K)
    assert (zq[100:164] == 0).all() and (zs[:, 100:164] == 0).all()
    assert (zq[164:] == gq[164:]).all() and (zq[:100] == gq[:100]).all()
    # bitwise stable from call to call
    gq2, gs2 = run(capi, cuda, case, M, I, K)
    assert np.array_equal(gq, gq2) and np.array_equal(gs.view(np.uint32), gs2.view(np.uint32))
    # the consumer: down projection of the fused output == down projection of the unfused path's output
    _, wd = fp8_sources(92, 8, 2560, I, w_std=0.02)
    D_q, D_s = oracle.quant_128x128(wd)
    dD, dDs = to_dev(cuda, D_q, D_s)
    Hq, Hs = to_dev(cuda, gq, gs)
    Y = torch.empty(M, 2560, device=cuda)
    capi.fp8_blockwise_mm_f32(Hq, Hs, dD, dDs, Y, M, 2560, I)
    # unfused: plain GEMM with fp32 output, SwiGLU in torch fp32, 1x128 quantiser, same down projection
    dA, dAs, dB, dBs = to_dev(cuda, *case)
    acc = torch.empty(M, 2 * I, device=cuda)
    capi.fp8_blockwise_mm_f32(dA, dAs, dB, dBs, acc, M, 2 * I, K)
    h = torch.nn.functional.silu(acc[:, :I]) * acc[:, I:]
    Uq = torch.empty(M, I, dtype=torch.uint8, device=cuda)
    Us = torch.empty(I // 128, M, device=cuda)
    capi.fp8_quant_1x128(h.contiguous(), Uq, Us, M, I)
    Y2 = torch.empty(M, 2560, device=cuda)
    capi.fp8_blockwise_mm_f32(Uq, Us, dD, dDs, Y2, M, 2560, I)
    torch.cuda.synchronize()
    capi.check_status()
    # the two activations differ only where an e4m3 rounding flipped: a few bytes in a thousand
    assert float((Uq == Hq).float().mean()) > 0.995
    assert float((Y - Y2).abs().max()) <= 2e-3 * float(Y2.abs().max())


@pytest.mark.parametrize("M", [1, 16, 33, 64])
@pytest.mark.parametrize("IK", [(9728, 2560), (256, 1024)])
def test_swiglu_decode_sized(capi, oracle, cuda, M, IK):
    # M <= 64 with enough scratch: the weight-streaming decode kernel + a small SwiGLU/quantise kernel (2 launches);
    # without scratch the 256-row kernel (1 launch).  Both against the oracle, and against each other.
    I, K = IK
    case = make_case(oracle, 93 + M, M, I, K)
    capi.clear_workspace()
    gq1, gs1 = run(capi, cuda, case, M, I, K, launches=1)
    check(oracle, case, gq1, gs1)
    capi.ensure_swiglu_workspace(M, I, K)
    gq2, gs2 = run(capi, cuda, case, M, I, K, launches=2)
    check(oracle, case, gq2, gs2)
    ok = gs1 > 0
    assert (np.abs(gs2[ok] / gs1[ok] - 1) <= 2e-5).all()
    assert (gq1 == gq2).mean() > 0.99
    gq3, gs3 = run(capi, cuda, case, M, I, K, launches=2)
    assert np.array_equal(gq2, gq3) and np.array_equal(gs2.view(np.uint32), gs3.view(np.uint32))


def test_swiglu_argument_errors(capi, cuda):
    z8 = torch.zeros(256, 256, dtype=torch.uint8, device=cuda)
    zf = torch.zeros(256, 256, device=cuda)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp8_blockwise_mm_swiglu(z8, zf, z8, zf, z8, zf, 128, 100, 128)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp8_blockwise_mm_swiglu(z8, zf, z8, zf, z8, zf, 128, 128, 64)
