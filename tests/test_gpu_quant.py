"""Bit-exact parity of the sm_100a blockwise quantisers with the oracle
(integer/byte outputs and IEEE-divided scales: no tolerance)."""
import numpy as np
import pytest
import torch

from helpers import fp8_sources

pytestmark = pytest.mark.gpu


def gpu_quant_1x128(capi, cuda, x):
    M, K = x.shape
    q = torch.full((M, K), 0xAA, dtype=torch.uint8, device=cuda)
    s = torch.full((K // 128, M), float("nan"), dtype=torch.float32, device=cuda)
    capi.fp8_quant_1x128(torch.from_numpy(x).to(cuda), q, s, M, K)
    torch.cuda.synchronize()
    return q.cpu().numpy(), s.cpu().numpy()


def gpu_quant_128x128(capi, cuda, w):
    R, C = w.shape
    q = torch.full((R, C), 0xAA, dtype=torch.uint8, device=cuda)
    s = torch.full((R // 128, C // 128), float("nan"), dtype=torch.float32, device=cuda)
    capi.fp8_quant_128x128(torch.from_numpy(w).to(cuda), q, s, R, C)
    torch.cuda.synchronize()
    return q.cpu().numpy(), s.cpu().numpy()


@pytest.mark.parametrize("shape", [(1, 128), (16, 2560), (33, 384), (64, 9728), (257, 1024), (1000, 512)])
def test_quant_1x128_bit_exact(capi, oracle, cuda, shape):
    x, _ = fp8_sources(30, shape[0], 128, shape[1])
    if shape[0] > 3:
        x[3, :128] = 0.0          # all-zero group
        x[2, 5] = 3.0e38          # huge value: scale near the top of fp32
        x[1, :128] *= 1e-30       # tiny group: scale is subnormal-sized
    q, s = gpu_quant_1x128(capi, cuda, x)
    oq, os_ = oracle.quant_1x128(x)
    assert (s.view(np.uint32) == os_.view(np.uint32)).all()
    assert (q == oq).all()


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (2560, 4096), (1024, 640)])
def test_quant_128x128_bit_exact(capi, oracle, cuda, shape):
    _, w = fp8_sources(31, 8, shape[0], shape[1], w_std=0.02)
    w[:128, :128] = 0.0
    q, s = gpu_quant_128x128(capi, cuda, w)
    oq, os_ = oracle.quant_128x128(w)
    assert (s.view(np.uint32) == os_.view(np.uint32)).all()
    assert (q == oq).all()


def test_full_size_quant_properties(capi, cuda):
    # 4096 x 4096 (the FP8 headline config): every group's largest code is +-448 and the
    # scale array is exactly amax/448 computed by torch in fp32
    M = K = 4096
    g = torch.Generator(device=cuda).manual_seed(32)
    x = torch.randn(M, K, device=cuda, generator=g)
    q = torch.empty(M, K, dtype=torch.uint8, device=cuda)
    s = torch.empty(K // 128, M, dtype=torch.float32, device=cuda)
    capi.fp8_quant_1x128(x, q, s, M, K)
    amax = x.view(M, K // 128, 128).abs().amax(dim=2)
    assert torch.equal(s.t().contiguous(), amax / torch.full_like(amax, 448.0))  # tensor / tensor: IEEE division
    codes = (q.view(M, K // 128, 128) & 0x7F).amax(dim=2)
    assert bool((codes == 0x7E).all())
    wq = torch.empty(M, K, dtype=torch.uint8, device=cuda)
    ws = torch.empty(M // 128, K // 128, dtype=torch.float32, device=cuda)
    capi.fp8_quant_128x128(x, wq, ws, M, K)
    bmax = x.view(M // 128, 128, K // 128, 128).abs().amax(dim=(1, 3))
    assert torch.equal(ws, bmax / torch.full_like(bmax, 448.0))
    # torch's own e4m3 conversion agrees with the bytes (same RN-even, saturating rule)
    deq_in = (x.view(M // 128, 128, K // 128, 128) / ws.view(M // 128, 1, K // 128, 1)).view(M, K)
    assert torch.equal(deq_in.to(torch.float8_e4m3fn).view(torch.uint8), wq)
    capi.check_status()


def test_quant_errors(capi, cuda):
    x = torch.zeros(4, 100, device=cuda)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp8_quant_1x128(x, torch.zeros(4, 100, dtype=torch.uint8, device=cuda), torch.zeros(1, 4, device=cuda), 4, 100)
