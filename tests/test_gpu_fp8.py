"""Parity of the sm_100a FP8 blockwise GEMM (through the C ABI) with the oracle.

Gates (from the task statement):
  * accumulator (fp32-output entry point): within 4e-6 * row amax of the fp64
    ground truth T0 of the quantised operands (accumulation-order noise only);
  * fused output: C_s and C_q are EXACTLY what the quantisation rule gives for
    the kernel's own accumulator (scales bit-exact from identical absmax);
  * de-quantised C: per element within (the oracle's own error against T0, which
    tests/golden pins as equal to the reference kernel's error) + 1 e4m3 ulp * scale.
"""
import numpy as np
import pytest
import torch

from helpers import e4m3_ulp, fp8_sources

pytestmark = pytest.mark.gpu

QWEN3_4B = [(6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728)]


def to_dev(cuda, *arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).to(cuda) for a in arrs]


def gpu_mm(capi, cuda, A_q, A_s, B_q, B_s, workspace=True):
    M, K = A_q.shape
    N = B_q.shape[0]
    dA, dAs, dB, dBs = to_dev(cuda, A_q, A_s, B_q, B_s)
    if workspace:
        capi.ensure_workspace(M, N, K)
    Cq = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
    Cs = torch.full((N // 128, M), float("nan"), dtype=torch.float32, device=cuda)
    Cf = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda)
    capi.fp8_blockwise_mm(dA, dAs, dB, dBs, Cq, Cs, M, N, K)
    capi.fp8_blockwise_mm_f32(dA, dAs, dB, dBs, Cf, M, N, K)
    torch.cuda.synchronize()
    capi.check_status()
    return Cq.cpu().numpy(), Cs.cpu().numpy(), Cf.cpu().numpy()


def check_against_oracle(oracle, A_q, A_s, B_q, B_s, gq, gs, gf, rows=None):
    M, N = gq.shape
    r0, n = (0, M) if rows is None else rows
    t0 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True, row0=r0, rows=n)
    t1 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s, row0=r0, rows=n)
    gq, gf, gs_rows = gq[r0:r0 + n], gf[r0:r0 + n], gs[:, r0:r0 + n]
    row_amax = np.abs(t0).max(axis=1, keepdims=True) + 1e-30
    # 1. accumulator
    assert (np.abs(gf - t0) <= 4e-6 * row_amax).all(), float((np.abs(gf - t0) / row_amax).max())
    assert (np.abs(t1 - t0) <= 4e-6 * row_amax).all()
    # 2. the fused output is the quantisation rule applied to the kernel's own accumulator, bit for bit
    q_rule, s_rule = oracle.c_quant_1x128(gf)
    assert (gs_rows.view(np.uint32) == s_rule.view(np.uint32)).all()
    assert (gq == q_rule).all()
    # 3. de-quantised values against the ground truth
    o_q, o_s = oracle.c_quant_1x128(t1)
    deq = oracle.e4m3_decode(gq) * np.repeat(gs_rows.T, 128, axis=1)
    o_deq = oracle.e4m3_decode(o_q) * np.repeat(o_s.T, 128, axis=1)
    scale_e = np.repeat(gs_rows.T, 128, axis=1).astype(np.float64)
    ulp = e4m3_ulp(oracle.e4m3_decode(gq)) * scale_e
    assert (np.abs(deq - t0) <= np.abs(o_deq - t0) + ulp + 1e-30).all()
    # scales within accumulation noise of the oracle's, bytes overwhelmingly identical
    ok = o_s > 0
    assert (np.abs(gs_rows[ok] / o_s[ok] - 1) <= 4e-6).all()
    assert (gq == o_q).mean() > 0.99


def make_case(oracle, seed, M, N, K, w_std=0.02):
    x, w = fp8_sources(seed, M, N, K, w_std=w_std)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    return A_q, A_s, B_q, B_s


@pytest.mark.parametrize("shape", [(128, 256, 128), (128, 128, 128), (256, 512, 512), (200, 384, 256), (129, 640, 1280),
                                   (512, 1152, 384)])
def test_general_kernel_small_shapes(capi, oracle, cuda, shape):
    M, N, K = shape
    case = make_case(oracle, 40, M, N, K)
    gq, gs, gf = gpu_mm(capi, cuda, *case)
    check_against_oracle(oracle, *case, gq, gs, gf)


@pytest.mark.parametrize("M", [1, 2, 15, 16, 17, 33, 64])
@pytest.mark.parametrize("NK", [(256, 1024), (384, 128), (2560, 4096), (19072, 256), (37888, 128), (25600, 512)])
def test_decode_kernel_ragged_m(capi, oracle, cuda, M, NK):
    """Among the shapes: 149 groups x 2 K-blocks (one whole group per CTA plus one left-over group cut in two),
    296 groups x 1 (two whole groups per CTA, nothing cut), 200 groups x 4 (one whole group per CTA and 52
    left-over groups cut into pieces of one or two K-blocks that cross group boundaries)."""
    N, K = NK
    case = make_case(oracle, 41 + M, M, N, K)
    gq, gs, gf = gpu_mm(capi, cuda, *case)
    check_against_oracle(oracle, *case, gq, gs, gf)


@pytest.mark.parametrize("M", [1, 16, 64])
@pytest.mark.parametrize("NK", QWEN3_4B)
def test_qwen3_4b_decode_shapes(capi, oracle, cuda, M, NK):
    N, K = NK
    case = make_case(oracle, 50, M, N, K)
    gq, gs, gf = gpu_mm(capi, cuda, *case)
    check_against_oracle(oracle, *case, gq, gs, gf)


def test_decode_without_workspace_uses_general_kernel(capi, oracle, cuda):
    # no scratch registered -> the library must still compute (general kernel), never fail or fall back to a CPU
    case = make_case(oracle, 42, 16, 512, 1024)
    capi.clear_workspace()
    gq, gs, gf = gpu_mm(capi, cuda, *case, workspace=False)
    check_against_oracle(oracle, *case, gq, gs, gf)
    gq2, gs2, gf2 = gpu_mm(capi, cuda, *case, workspace=True)
    check_against_oracle(oracle, *case, gq2, gs2, gf2)
    # split-K changes only the order of the fp32 promotion sums
    assert np.abs(gf - gf2).max() <= 4e-6 * np.abs(gf).max()


def test_decode_repeated_calls_are_bitwise_stable(capi, oracle, cuda):
    # the arrival counters reset themselves and partials are summed in a fixed order
    M, N, K = 16, 2560, 9728
    A_q, A_s, B_q, B_s = make_case(oracle, 43, M, N, K)
    dA, dAs, dB, dBs = to_dev(cuda, A_q, A_s, B_q, B_s)
    capi.ensure_workspace(M, N, K)
    outs = []
    for _ in range(5):
        Cq = torch.zeros(M, N, dtype=torch.uint8, device=cuda)
        Cs = torch.zeros(N // 128, M, dtype=torch.float32, device=cuda)
        capi.fp8_blockwise_mm(dA, dAs, dB, dBs, Cq, Cs, M, N, K)
        outs.append((Cq, Cs))
    torch.cuda.synchronize()
    for Cq, Cs in outs[1:]:
        assert torch.equal(Cq, outs[0][0]) and torch.equal(Cs, outs[0][1])
    capi.check_status()


# Shapes whose last wave of 256x256 tiles is shared out K-block by K-block when scratch is registered:
# few tiles with a long K (every tile has many contributors), ragged M and N, and several full waves
# followed by a partial one.
SPLIT_SHAPES = [(256, 512, 4096), (384, 640, 4096), (300, 1280, 3584), (1024, 2048, 4096), (2304, 4352, 4096)]


@pytest.mark.parametrize("shape", SPLIT_SHAPES)
def test_split_last_wave(capi, oracle, cuda, shape):
    M, N, K = shape
    case = make_case(oracle, 44, M, N, K)
    rows = None if M <= 1024 else (M - 700, 700)
    capi.clear_workspace()
    n0 = capi.split_launch_count()
    gq, gs, gf = gpu_mm(capi, cuda, *case, workspace=False)
    assert capi.split_launch_count() == n0
    check_against_oracle(oracle, *case, gq, gs, gf, rows=rows)
    gq2, gs2, gf2 = gpu_mm(capi, cuda, *case, workspace=True)
    # the split does take place for these shapes (both entry points), otherwise this test checks nothing
    assert capi.split_launch_count() == n0 + 2
    check_against_oracle(oracle, *case, gq2, gs2, gf2, rows=rows)
    # splitting changes only the order of the fp32 promotion sums
    assert np.abs(gf - gf2).max() <= 4e-6 * np.abs(gf).max()
    # bitwise stable from call to call: counters reset themselves, pieces are added in a fixed order
    gq3, gs3, gf3 = gpu_mm(capi, cuda, *case, workspace=True)
    assert np.array_equal(gq2, gq3) and np.array_equal(gs2.view(np.uint32), gs3.view(np.uint32)) and np.array_equal(gf2, gf3)


@pytest.mark.parametrize("M", [1, 16, 64])
def test_decode_launch_chain_with_static_weights(capi, oracle, cuda, M):
    # Back-to-back launches without synchronisation, each using the previous one's stream position: with the
    # static-weights promise a launch prefetches its weights while the one before it is finishing; results
    # must be what the un-promised chain gives, bit for bit, and right.
    N, K = 2560, 4096
    cases = [make_case(oracle, 80 + i, M, N, K) for i in range(3)]
    dev = [to_dev(cuda, *c) for c in cases]
    capi.ensure_workspace(M, N, K)

    def chain():
        outs = []
        for rep in range(4):
            for dA, dAs, dB, dBs in dev:
                Cq = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
                Cs = torch.full((N // 128, M), float("nan"), device=cuda)
                outs.append((Cq, Cs))
        i = 0
        for rep in range(4):
            for dA, dAs, dB, dBs in dev:
                capi.fp8_blockwise_mm(dA, dAs, dB, dBs, outs[i][0], outs[i][1], M, N, K)
                i += 1
        torch.cuda.synchronize()
        capi.check_status()
        return outs

    plain = chain()
    capi.set_static_weights(True)
    try:
        promised = chain()
    finally:
        capi.set_static_weights(False)
    for (q0, s0), (q1, s1) in zip(plain, promised):
        assert torch.equal(q0, q1) and torch.equal(s0, s1)
    for i, case in enumerate(cases):
        Cf = torch.empty(M, N, device=cuda)
        capi.fp8_blockwise_mm_f32(*dev[i], Cf, M, N, K)
        torch.cuda.synchronize()
        check_against_oracle(oracle, *case, promised[i][0].cpu().numpy(), promised[i][1].cpu().numpy(), Cf.cpu().numpy())


@pytest.mark.parametrize("shape", [(128, 2560, 4096), (65, 512, 2048), (100, 4096, 1024)])
def test_mid_m_few_tiles_take_the_pair_kernel_with_scratch(capi, oracle, cuda, shape):
    # 65..128 rows, tiles on at most half of the SMs: single-CTA kernel without scratch, pair kernel (whose tiles
    # are cut along K) with it; both against the oracle, and within the order of fp32 sums of each other
    M, N, K = shape
    case = make_case(oracle, 45, M, N, K)
    capi.clear_workspace()
    assert "fp8_blockwise_gemm_kernel" in capi.describe_plan("fp8", M, N, K)
    gq, gs, gf = gpu_mm(capi, cuda, *case, workspace=False)
    check_against_oracle(oracle, *case, gq, gs, gf)
    capi.ensure_workspace(M, N, K)
    assert "fp8_blockwise_gemm_pair_kernel" in capi.describe_plan("fp8", M, N, K)
    gq2, gs2, gf2 = gpu_mm(capi, cuda, *case, workspace=True)
    check_against_oracle(oracle, *case, gq2, gs2, gf2)
    assert np.abs(gf - gf2).max() <= 4e-6 * np.abs(gf).max()


def gpu_c_quant(acc):
    """The output quantisation rule in torch fp32 on the GPU (for full-size property checks)."""
    M, N = acc.shape
    g = acc.view(M, N // 128, 128)
    amax = g.abs().amax(dim=2, keepdim=True)
    c448 = torch.full_like(amax, 448.0)  # tensor / tensor is an IEEE division; tensor / python-scalar multiplies by 1/448
    scale = amax / c448
    inv = torch.where(amax > 0, c448 / amax, torch.zeros_like(amax))
    q = (g * inv).to(torch.float8_e4m3fn).view(torch.uint8).view(M, N)
    return q, scale.squeeze(2).t().contiguous()


def full_size_case(capi, cuda, M, N, K, seed, w_std):
    g = torch.Generator(device=cuda).manual_seed(seed)
    x = torch.randn(M, K, device=cuda, generator=g)
    w = torch.randn(N, K, device=cuda, generator=g) * w_std
    A_q = torch.empty(M, K, dtype=torch.uint8, device=cuda)
    A_s = torch.empty(K // 128, M, device=cuda)
    B_q = torch.empty(N, K, dtype=torch.uint8, device=cuda)
    B_s = torch.empty(N // 128, K // 128, device=cuda)
    capi.fp8_quant_1x128(x, A_q, A_s, M, K)
    capi.fp8_quant_128x128(w, B_q, B_s, N, K)
    return A_q, A_s, B_q, B_s


@pytest.mark.parametrize("shape", [(4096, 4096, 4096, 1.0), (4096, 6144, 2560, 0.02), (4096, 2560, 9728, 0.02)])
def test_full_size_properties_and_sampled_rows(capi, oracle, cuda, shape):
    M, N, K, w_std = shape
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, 60, w_std)
    capi.ensure_workspace(M, N, K)
    Cq = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
    Cs = torch.full((N // 128, M), float("nan"), device=cuda)
    Cf = torch.full((M, N), float("nan"), device=cuda)
    capi.fp8_blockwise_mm(A_q, A_s, B_q, B_s, Cq, Cs, M, N, K)
    capi.fp8_blockwise_mm_f32(A_q, A_s, B_q, B_s, Cf, M, N, K)
    # (a) fused output == rule(own accumulator), everywhere, bit for bit
    q_rule, s_rule = gpu_c_quant(Cf)
    assert torch.equal(Cs, s_rule)
    assert torch.equal(Cq, q_rule)
    # (b) linearity: doubling the activation scales doubles the accumulator and the output scales exactly
    Cq2 = torch.empty_like(Cq)
    Cs2 = torch.empty_like(Cs)
    capi.fp8_blockwise_mm(A_q, A_s * 2, B_q, B_s, Cq2, Cs2, M, N, K)
    assert torch.equal(Cq2, Cq) and torch.equal(Cs2, Cs * 2)
    # (c) erasure: zeroed activation rows give zero bytes and zero scales (the defined all-zero case)
    A_q0 = A_q.clone()
    A_q0[100:228] = 0
    capi.fp8_blockwise_mm(A_q0, A_s, B_q, B_s, Cq2, Cs2, M, N, K)
    assert bool((Cq2[100:228] == 0).all()) and bool((Cs2[:, 100:228] == 0).all())
    assert torch.equal(Cq2[228:], Cq[228:]) and torch.equal(Cq2[:100], Cq[:100])
    torch.cuda.synchronize()
    capi.check_status()
    # (d) sampled whole rows against the CPU oracle
    hA_q, hA_s, hB_q, hB_s = (t.cpu().numpy() for t in (A_q, A_s, B_q, B_s))
    gq, gs, gf = Cq.cpu().numpy(), Cs.cpu().numpy(), Cf.cpu().numpy()
    for r0 in (0, 127, 2049, M - 4):
        check_against_oracle(oracle, hA_q, hA_s, hB_q, hB_s, gq, gs, gf, rows=(r0, 4))


def test_reference_launcher_errors(capi, cuda):
    z8 = torch.zeros(128, 128, dtype=torch.uint8, device=cuda)
    zf = torch.zeros(128, 128, device=cuda)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp8_blockwise_mm(z8, zf, z8, zf, z8, zf, 128, 100, 128)
