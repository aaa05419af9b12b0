"""RMSNorm fused in front of the 1x128 activation quantiser, against the oracle.

A floating-point kernel (the sum of squares is reduced in a different order than on the CPU and the reciprocal
square root is the hardware's correctly rounded one), so the gate is a tolerance, stated here: the normalised
value may differ from the fp64 truth by 4e-7 relative (three fp32 roundings and the sum's order).  On the outputs:
scales within 1e-6 relative of the oracle's, bytes identical except where a value sits on an e4m3 rounding
boundary (> 99.9 %), de-quantised values within the oracle's own error + 1 e4m3 ulp * scale; and the
composition property: the result equals the plain quantiser applied to the normalised tensor computed in torch."""
import numpy as np
import pytest
import torch

from helpers import e4m3_ulp

pytestmark = pytest.mark.gpu


def run(capi, cuda, x, w, eps):
    M, K = x.shape
    q = torch.full((M, K), 0xAA, dtype=torch.uint8, device=cuda)
    s = torch.full((K // 128, M), float("nan"), device=cuda)
    before = capi.launch_count()
    capi.fp8_rmsnorm_quant_1x128(torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda), eps, q, s, M, K)
    torch.cuda.synchronize()
    capi.check_status()
    assert capi.launch_count() == before + 1
    return q.cpu().numpy(), s.cpu().numpy()


@pytest.mark.parametrize("shape", [(1, 128), (16, 2560), (33, 384), (64, 9728), (257, 1024), (512, 18944)])
def test_rmsnorm_quant_against_oracle(capi, oracle, cuda, shape):
    M, K = shape
    rng = np.random.default_rng(100 + M)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.1, 30.0, (M, 1))).astype(np.float32)
    w = rng.uniform(0.5, 1.5, K).astype(np.float32)
    if M > 3:
        x[3] = 0.0  # an all-zero row: y = 0, scale 0, zero bytes (eps keeps the rsqrt finite)
    eps = 1e-6
    gq, gs = run(capi, cuda, x, w, eps)
    oq, os_, y32, y64 = oracle.rmsnorm_quant_1x128(x, w, eps)
    assert np.isfinite(gs).all()
    ok = os_ > 0
    assert (np.abs(gs[ok] / os_[ok] - 1) <= 1e-6).all(), float(np.abs(gs[ok] / os_[ok] - 1).max())
    assert (gs[~ok] == 0).all()
    assert (gq == oq).mean() > 0.999
    scale_e = np.repeat(gs.T, 128, axis=1).astype(np.float64)
    deq = oracle.e4m3_decode(gq) * scale_e
    o_deq = oracle.e4m3_decode(oq) * np.repeat(os_.T, 128, axis=1).astype(np.float64)
    ulp = e4m3_ulp(oracle.e4m3_decode(gq)) * scale_e
    assert (np.abs(deq - y64) <= np.abs(o_deq - y64) + ulp + 4e-7 * np.abs(y64) + 1e-30).all()
    if M > 3:
        assert (gq[3] == 0).all() and (gs[:, 3] == 0).all()


def test_rmsnorm_quant_equals_norm_then_quant(capi, cuda):
    M, K = 4096, 2560
    g = torch.Generator(device=cuda).manual_seed(101)
    x = torch.randn(M, K, device=cuda, generator=g) * 3
    w = torch.rand(K, device=cuda, generator=g) + 0.5
    q = torch.empty(M, K, dtype=torch.uint8, device=cuda)
    s = torch.empty(K // 128, M, device=cuda)
    capi.fp8_rmsnorm_quant_1x128(x, w, 1e-6, q, s, M, K)
    y = x * torch.rsqrt((x.double() ** 2).mean(dim=1, keepdim=True).float() + 1e-6) * w
    q2 = torch.empty_like(q)
    s2 = torch.empty_like(s)
    capi.fp8_quant_1x128(y.contiguous(), q2, s2, M, K)
    torch.cuda.synchronize()
    capi.check_status()
    assert bool(((s - s2).abs() <= 1e-6 * s2.abs()).all())
    assert float((q == q2).float().mean()) > 0.999


def test_rmsnorm_quant_argument_errors(capi, cuda):
    x = torch.zeros(4, 256, device=cuda)
    w = torch.ones(256, device=cuda)
    q = torch.zeros(4, 256, dtype=torch.uint8, device=cuda)
    s = torch.zeros(2, 4, device=cuda)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp8_rmsnorm_quant_1x128(x, w, 1e-6, q, s, 4, 200)
    with pytest.raises(RuntimeError, match="eps"):
        capi.fp8_rmsnorm_quant_1x128(x, w, -1.0, q, s, 4, 256)
