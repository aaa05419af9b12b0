"""qkv projection with the per-head q/k RMSNorm and the rotary embedding fused into the epilogue, against the oracle.

A floating-point epilogue (a reciprocal square root per head, two products and a sum per element), so the gate is
a tolerance, stated here: the fp32 y the kernel quantises may differ from the fp64 truth by 3e-5 of its head's
largest |y| (GEMM accumulation noise 4e-6 as for the plain kernel, carried through the normalisation, which keeps
relative errors, and the rotation, which mixes two values of similar size; plus the approximate reciprocal square
root, 2^-22 relative).  On the outputs: scales within 3e-5 relative of the oracle's, de-quantised values within
the oracle's own error + 1 e4m3 ulp * scale + that bound, bytes overwhelmingly identical.  Two properties are
bit-exact: value heads equal the plain GEMM's output, and with identity angles (cos 1, sin 0) and no norm weights
the whole output equals the plain GEMM's.

Budget of the approximate intrinsic in the fused epilogue (CUDA's documented maximum error): `rsqrtf` is 2 ulp =
2.4e-7 relative, applied once per head as a common factor of its 128 values (the small hook kernel of the
M <= 64 path uses the correctly rounded `__fsqrt_rn` / `__frcp_rn`).  The sum of squares is taken in four FMA
chains (<= 128 * 2^-24 = 7.6e-6 relative in the worst case, 1e-6 typical) and halves under the square root.  Both
are far inside the 3e-5 gate, whose larger part is the accumulation noise of the GEMM carried through the
rotation."""
import numpy as np
import pytest
import torch

from helpers import e4m3_ulp, fp8_sources
from test_gpu_fp8 import to_dev

pytestmark = pytest.mark.gpu

EPS = 1e-6


def make_case(oracle, seed, M, n_q, n_kv, K, weights=True, positions=4096):
    N = (n_q + 2 * n_kv) * 128
    x, w = fp8_sources(seed, M, N, K, w_std=0.05)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    rng = np.random.default_rng(seed + 1000)
    pos = rng.integers(0, positions, size=M).astype(np.int32)
    inv_freq = 1.0 / (1e6 ** (np.arange(64, dtype=np.float64) / 64))
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    q_w = (1 + 0.2 * rng.standard_normal(128)).astype(np.float32) if weights else None
    k_w = (1 + 0.2 * rng.standard_normal(128)).astype(np.float32) if weights else None
    return dict(gemm=(A_q, A_s, B_q, B_s), pos=pos, cos=cos, sin=sin, q_w=q_w, k_w=k_w, n_q=n_q, n_kv=n_kv, M=M, N=N, K=K)


def run(capi, cuda, c, launches=1):
    M, N, K = c["M"], c["N"], c["K"]
    dA, dAs, dB, dBs = to_dev(cuda, *c["gemm"])
    t = lambda a: None if a is None else torch.from_numpy(a).to(cuda)
    Cq = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
    Cs = torch.full((N // 128, M), float("nan"), device=cuda)
    before = capi.launch_count()
    capi.fp8_blockwise_mm_qk_norm_rope(dA, dAs, dB, dBs, Cq, Cs, t(c["pos"]), t(c["cos"]), t(c["sin"]), t(c["q_w"]),
                                       t(c["k_w"]), EPS, c["n_q"], c["n_kv"], M, N, K)
    torch.cuda.synchronize()
    capi.check_status()
    assert capi.launch_count() == before + launches
    return Cq.cpu().numpy(), Cs.cpu().numpy()


def plain(capi, cuda, c):
    M, N, K = c["M"], c["N"], c["K"]
    dA, dAs, dB, dBs = to_dev(cuda, *c["gemm"])
    Cq = torch.empty((M, N), dtype=torch.uint8, device=cuda)
    Cs = torch.empty((N // 128, M), device=cuda)
    capi.fp8_blockwise_mm(dA, dAs, dB, dBs, Cq, Cs, M, N, K)
    torch.cuda.synchronize()
    return Cq.cpu().numpy(), Cs.cpu().numpy()


def check(oracle, c, gq, gs, rows=None):
    r0, n = (0, c["M"]) if rows is None else rows
    oq, os_, y32, y64 = oracle.fp8_blockwise_mm_qk_norm_rope(*c["gemm"], c["pos"], c["cos"], c["sin"], c["q_w"], c["k_w"],
                                                             EPS, c["n_q"], c["n_kv"], row0=r0, rows=n)
    gq, gs = gq[r0:r0 + n], gs[:, r0:r0 + n]
    assert np.isfinite(gs).all()
    head_amax = np.repeat(np.abs(y64).reshape(n, -1, 128).max(axis=2), 128, axis=1) + 1e-30
    ok = os_ > 0
    assert (np.abs(gs[ok] / os_[ok] - 1) <= 3e-5).all(), float(np.abs(gs[ok] / os_[ok] - 1).max())
    scale_e = np.repeat(gs.T, 128, axis=1).astype(np.float64)
    deq = oracle.e4m3_decode(gq) * scale_e
    o_deq = oracle.e4m3_decode(oq) * np.repeat(os_.T, 128, axis=1).astype(np.float64)
    ulp = e4m3_ulp(oracle.e4m3_decode(gq)) * scale_e
    assert (np.abs(deq - y64) <= np.abs(o_deq - y64) + ulp + 3e-5 * head_amax).all()
    assert (gq == oq).mean() > 0.99


@pytest.mark.parametrize("shape", [(256, 2, 1, 256), (200, 4, 2, 512), (1, 2, 1, 384), (640, 3, 3, 256)])
@pytest.mark.parametrize("weights", [True, False])
def test_small_shapes(capi, oracle, cuda, shape, weights):
    M, n_q, n_kv, K = shape
    c = make_case(oracle, 70, M, n_q, n_kv, K, weights=weights)
    capi.clear_workspace()  # the fused 256-row kernel for every M
    gq, gs = run(capi, cuda, c)
    check(oracle, c, gq, gs)
    # value heads are the plain GEMM's, bit for bit
    pq, ps = plain(capi, cuda, c)
    v0 = (n_q + n_kv) * 128
    assert (gq[:, v0:] == pq[:, v0:]).all() and (gs[n_q + n_kv:] == ps[n_q + n_kv:]).all()


def test_identity_angles_without_weights_equal_the_plain_gemm(capi, oracle, cuda):
    c = make_case(oracle, 71, 300, 4, 2, 512, weights=False)
    c["cos"] = np.ones_like(c["cos"])
    c["sin"] = np.zeros_like(c["sin"])
    capi.clear_workspace()
    gq, gs = run(capi, cuda, c)
    pq, ps = plain(capi, cuda, c)
    assert (gq == pq).all() and (gs == ps).all()


def test_registered_scratch_does_not_cut_tiles(capi, oracle, cuda):
    # few tiles with a long K: the plain GEMM cuts them along K when scratch is registered, the hooked kernel
    # keeps whole tiles (it has no code for chunks) and gives the same bytes with and without scratch
    c = make_case(oracle, 74, 300, 2, 1, 4096)
    capi.clear_workspace()
    gq, gs = run(capi, cuda, c)
    check(oracle, c, gq, gs)
    capi.ensure_workspace(c["M"], c["N"], c["K"])
    n0 = capi.split_launch_count()
    plain(capi, cuda, c)
    assert capi.split_launch_count() == n0 + 1
    gq2, gs2 = run(capi, cuda, c)
    assert capi.split_launch_count() == n0 + 1
    assert (gq2 == gq).all() and (gs2 == gs).all()


def test_qwen3_4b_qkv_prefill(capi, oracle, cuda):
    # 32 query + 8 key + 8 value heads of 128 over hidden size 2560, with and without registered scratch
    # (which this kernel does not use)
    c = make_case(oracle, 72, 1024, 32, 8, 2560)
    capi.clear_workspace()
    gq, gs = run(capi, cuda, c)
    check(oracle, c, gq, gs, rows=(1016, 8))
    check(oracle, c, gq, gs, rows=(301, 4))
    capi.ensure_workspace(c["M"], c["N"], c["K"])
    gq2, gs2 = run(capi, cuda, c)
    assert (gq2 == gq).all() and (gs2 == gs).all()
    gq3, gs3 = run(capi, cuda, c)
    assert (gq2 == gq3).all() and (gs2 == gs3).all()  # bitwise stable from call to call


@pytest.mark.parametrize("M", [1, 4, 64])
def test_decode_sized(capi, oracle, cuda, M):
    # with scratch: the weight-streaming decode kernel + the small hook kernel (two launches)
    c = make_case(oracle, 73, M, 32, 8, 2560)
    capi.ensure_qk_norm_rope_workspace(c["M"], c["N"], c["K"])
    gq, gs = run(capi, cuda, c, launches=2)
    check(oracle, c, gq, gs)


def test_argument_errors(capi, cuda):
    c = dict(M=128, N=512, K=256)
    z8 = torch.zeros(128 * 512, dtype=torch.uint8, device=cuda)
    zf = torch.zeros(128 * 512, dtype=torch.float32, device=cuda)
    zi = torch.zeros(128, dtype=torch.int32, device=cuda)
    zt = torch.zeros(16, 64, dtype=torch.float32, device=cuda)
    with pytest.raises(RuntimeError, match="n_q_heads"):
        capi.fp8_blockwise_mm_qk_norm_rope(z8, zf, z8, zf, z8, zf, zi, zt, zt, None, None, EPS, 2, 2, 128, 512, 256)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp8_blockwise_mm_qk_norm_rope(z8, zf, z8, zf, z8, zf, zi, zt, zt, None, None, EPS, 2, 1, 128, 512, 200)
    with pytest.raises(RuntimeError, match=r"\[rows, 64\]"):
        capi.fp8_blockwise_mm_qk_norm_rope(z8, zf, z8, zf, z8, zf, zi, zf, zf, None, None, EPS, 2, 1, 128, 512, 256)


@pytest.mark.parametrize("M", [8, 256])
def test_positions_outside_the_tables_are_clamped_and_reported(capi, cuda, M):
    """The angle tables have `rows` rows; a position below 0 or at / beyond `rows` must not be used as an index.  The
    kernels (the fused epilogue for M > 64, the small hook kernel for M <= 64) clamp it to the nearest row, so the
    result equals the one for the clamped positions, and record code 0x201 in the status word."""
    N, K, n_q, n_kv, rows = 512, 256, 2, 1, 16
    g = torch.Generator(device=cuda).manual_seed(5)
    A = torch.randint(0, 120, (M, K), dtype=torch.uint8, device=cuda, generator=g)
    As = torch.rand(K // 128, M, device=cuda, generator=g)
    B = torch.randint(0, 120, (N, K), dtype=torch.uint8, device=cuda, generator=g)
    Bs = torch.rand(N // 128, K // 128, device=cuda, generator=g)
    ang = torch.rand(rows, 64, device=cuda, generator=g) * 6.28
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    pos = (torch.arange(M, device=cuda, dtype=torch.int32) % rows).contiguous()
    bad = pos.clone()
    bad[0], bad[M - 1] = -7, rows + 1000
    good = bad.clamp(0, rows - 1)
    capi.ensure_qk_norm_rope_workspace(M, N, K)
    out = []
    for p in (good, bad):
        Cq = torch.zeros(M, N, dtype=torch.uint8, device=cuda)
        Cs = torch.zeros(N // 128, M, device=cuda)
        capi.fp8_blockwise_mm_qk_norm_rope(A, As, B, Bs, Cq, Cs, p, cos, sin, None, None, EPS, n_q, n_kv, M, N, K)
        torch.cuda.synchronize()
        if p is good:
            capi.check_status()
        else:
            with pytest.raises(RuntimeError, match="0x201"):
                capi.check_status()
        out.append((Cq, Cs))
    assert torch.equal(out[0][0], out[1][0]) and torch.equal(out[0][1], out[1][1])
    capi.check_status()  # the word was cleared by the report
