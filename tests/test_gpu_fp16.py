"""Parity of the sm_100a FP16/BF16 GEMM (through the C ABI) with the oracle.

Tolerance (stated by the task for this floating-point kernel): relative error
<= 1e-3 of the fp64 product of the 16-bit inputs, with an absolute floor of
1e-3 * sqrt(K)/8 for results that cancel to nearly zero (the fp32 Kahan
reference GEMM of test/kahan.cu is checked against the same truth)."""
import numpy as np
import pytest
import torch

from helpers import fp16_inputs

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


def run_case(capi, oracle, cuda, M, N, K, dtype, seed, rows=None, scratch=None):
    """scratch: None = whatever is registered, False = none (whole tiles only), True = registered (the
    tiles of a partly filled last wave are cut along K)."""
    if scratch is True:
        capi.ensure_workspace(M, max(N, 128), max(K, 128))
    elif scratch is False:
        capi.clear_workspace()
    A, B = fp16_inputs(seed, M, N, K)
    if dtype == torch.float16:
        Ar, Br = oracle.from_f16_bits(oracle.to_f16_bits(A)), oracle.from_f16_bits(oracle.to_f16_bits(B))
    else:
        Ar, Br = oracle.from_bf16_bits(oracle.to_bf16_bits(A)), oracle.from_bf16_bits(oracle.to_bf16_bits(B))
    dA = torch.from_numpy(Ar).to(cuda).to(dtype)
    dB = torch.from_numpy(Br).to(cuda).to(dtype)
    dC = torch.full((M, N), float("nan"), dtype=dtype, device=cuda)
    before = capi.launch_count()
    capi.fp16_mm(dA, dB, dC, M, N, K)
    torch.cuda.synchronize()
    capi.check_status()
    assert capi.launch_count() == before + 1
    C = dC.float().cpu().numpy()
    assert np.isfinite(C).all(), "part of C was not written"
    if rows is None:
        row_sets = [(0, M)]
    else:
        row_sets = rows
    worst = 0.0
    out_ulp = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
    for r0, n in row_sets:
        exact = oracle.exact_gemm(Ar, Br, r0, n)
        got = C[r0:r0 + n]
        tol = (REL_TOL + out_ulp) * np.abs(exact) + 1e-3 * np.sqrt(K) / 8
        err = np.abs(got - exact)
        assert (err <= tol).all(), f"max err {err.max()} at rows {r0}:{r0+n}"
        big = np.abs(exact) > 0.05 * np.sqrt(K)
        if big.any():
            worst = max(worst, float((err[big] / np.abs(exact[big])).max()))
            # on well-conditioned elements the kernel must meet the pure relative gate
            lim = REL_TOL if dtype == torch.float16 else 2.0 ** -8
            assert worst <= lim
        # the named reference (fp32 Kahan) agrees with the same truth far inside the gate
        kahan = oracle.kahan_gemm(Ar, Br, r0, n)
        assert np.abs(kahan - exact).max() <= 1e-4 * max(1.0, np.abs(exact).max())
    return worst


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_config0_256_cubed_full(capi, oracle, cuda, dtype):
    run_case(capi, oracle, cuda, 256, 256, 256, dtype, seed=0)


@pytest.mark.parametrize("shape", [(128, 256, 64), (1, 8, 8), (7, 264, 136), (200, 520, 72), (129, 256, 1024),
                                   (384, 768, 40), (640, 1280, 320)])
def test_edge_and_ragged_shapes(capi, oracle, cuda, shape):
    M, N, K = shape
    run_case(capi, oracle, cuda, M, N, K, torch.float16, seed=1)


# Shapes whose last wave of 256x256 tiles is cut along K when scratch is registered: few tiles with a long
# K, ragged M / N, a K that is not a multiple of the 64-wide K-step, full waves followed by a partial one.
SPLIT_SHAPES = [(256, 512, 4096), (384, 640, 4096), (300, 1288, 3592), (2304, 4352, 4096)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SPLIT_SHAPES)
def test_split_last_wave(capi, oracle, cuda, shape, dtype):
    M, N, K = shape
    rows = None if M <= 512 else [(M - 300, 300)]
    n0 = capi.split_launch_count()
    run_case(capi, oracle, cuda, M, N, K, dtype, seed=5, rows=rows, scratch=False)
    assert capi.split_launch_count() == n0
    run_case(capi, oracle, cuda, M, N, K, dtype, seed=5, rows=rows, scratch=True)
    assert capi.split_launch_count() == n0 + 1


@pytest.mark.parametrize("shape", [(128, 2560, 4096), (65, 512, 8192), (100, 4096, 4104)])
def test_mid_m_few_tiles_take_the_pair_kernel_with_scratch(capi, oracle, cuda, shape):
    # 65..128 rows whose tiles would occupy at most half of the SMs: the single-CTA kernel without scratch,
    # the pair kernel (tiles cut along K) with it
    M, N, K = shape
    capi.clear_workspace()
    assert "fp16_gemm_kernel" in capi.describe_plan("fp16", M, N, K)
    run_case(capi, oracle, cuda, M, N, K, torch.float16, seed=8, scratch=False)
    capi.ensure_workspace(M, N, K)
    assert "fp16_gemm_pair_kernel" in capi.describe_plan("fp16", M, N, K)
    n0 = capi.split_launch_count()
    run_case(capi, oracle, cuda, M, N, K, torch.bfloat16, seed=8, scratch=True)
    assert capi.split_launch_count() == n0 + 1


def test_split_is_bitwise_stable(capi, cuda):
    # arrival counters reset themselves and the chunks are added in a fixed order
    M, N, K = 384, 640, 4096
    g = torch.Generator(device=cuda).manual_seed(6)
    A = torch.randn(M, K, device=cuda, generator=g).half()
    B = torch.randn(K, N, device=cuda, generator=g).half()
    capi.ensure_workspace(M, N, K)
    outs = []
    n0 = capi.split_launch_count()
    for _ in range(5):
        C = torch.empty(M, N, dtype=torch.float16, device=cuda)
        capi.fp16_mm(A, B, C, M, N, K)
        outs.append(C)
    torch.cuda.synchronize()
    capi.check_status()
    assert capi.split_launch_count() == n0 + 5
    for C in outs[1:]:
        assert torch.equal(C, outs[0])


def test_config1_4096_cubed_sampled(capi, oracle, cuda):
    # full size; 64 whole rows spread over the tiles plus the last row are checked on the CPU
    rows = [(r, 8) for r in (0, 120, 127 + 1, 1000, 2048 + 64, 3333, 4000, 4088)]
    run_case(capi, oracle, cuda, 4096, 4096, 4096, torch.float16, seed=2, rows=rows, scratch=True)


def test_full_size_linearity_and_identity(capi, cuda):
    # size-independent properties at 4096^3: A @ I == A exactly, and (2A) @ B == 2 (A @ B) exactly
    M = N = K = 4096
    g = torch.Generator(device=cuda).manual_seed(3)
    A = (torch.rand(M, K, device=cuda, generator=g) * 2 - 1).half()
    B = (torch.rand(K, N, device=cuda, generator=g) * 2 - 1).half()
    eye = torch.eye(K, device=cuda, dtype=torch.float16)
    C = torch.empty(M, N, device=cuda, dtype=torch.float16)
    capi.fp16_mm(A, eye, C, M, N, K)
    assert torch.equal(C, A)
    C1 = torch.empty_like(C)
    C2 = torch.empty_like(C)
    capi.fp16_mm(A, B, C1, M, N, K)
    capi.fp16_mm(A * 2, B, C2, M, N, K)
    normal = C1.abs() >= 2.0 ** -14  # a subnormal half result has fewer bits than its double
    assert torch.equal(C2[normal], (C1 * 2)[normal])
    assert float((C2.float() - 2 * C1.float()).abs().max()) <= 2.0 ** -24
    # run twice: bitwise reproducible
    capi.fp16_mm(A, B, C2, M, N, K)
    assert torch.equal(C2, C1)
    capi.check_status()


def test_reference_launcher_errors(capi, cuda):
    A = torch.zeros(256, 256, device=cuda, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp16_mm(A, A, A, 256, 250, 256)
    with pytest.raises(RuntimeError, match="T is not supported"):
        capi.fp16_mm(A.float(), A.float(), A.float(), 256, 256, 256)


def test_other_stream(capi, oracle, cuda):
    s = torch.cuda.Stream()
    A, B = fp16_inputs(4, 128, 256, 128)
    dA, dB = torch.from_numpy(A).to(cuda).half(), torch.from_numpy(B).to(cuda).half()
    dC = torch.zeros(128, 256, device=cuda, dtype=torch.float16)
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        capi.fp16_mm(dA, dB, dC, 128, 256, 128)
    s.synchronize()
    exact = oracle.exact_gemm(dA.float().cpu().numpy(), dB.float().cpu().numpy())
    assert np.abs(dC.float().cpu().numpy() - exact).max() <= 2e-3 * np.abs(exact).max()
