"""Bit-exact parity of the transpose (reference: src/base/base.cu:125-155, test
test/transpose_matrix__aligned_128_test.cc) on the reference test's own shapes."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(128, 128), (256, 384), (4096, 4096), (6144, 2048), (2048, 12288)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.uint8])
def test_transpose_bit_exact(capi, oracle, cuda, shape, dtype):
    M, N = shape
    g = torch.Generator(device=cuda).manual_seed(80)
    if dtype == torch.float32:
        src = torch.rand(M, N, device=cuda, generator=g) * 10 - 5
    else:
        src = torch.randint(0, 256, (M, N), dtype=torch.uint8, device=cuda, generator=g)
    dst = torch.zeros(N, M, dtype=dtype, device=cuda)
    capi.transpose_aligned_128(dst, src, M, N)
    torch.cuda.synchronize()
    assert torch.equal(dst, src.t().contiguous())
    if M * N <= 256 * 384:  # the small cases also against the CPU oracle
        assert (dst.cpu().numpy() == oracle.transpose(src.cpu().numpy())).all()
    # involution: transposing back restores the input
    back = torch.zeros_like(src)
    capi.transpose_aligned_128(back, dst, N, M)
    assert torch.equal(back, src)


def test_transpose_errors(capi, cuda):
    x = torch.zeros(128, 100, device=cuda)
    with pytest.raises(RuntimeError, match="can't be divided 128"):
        capi.transpose_aligned_128(torch.zeros(100, 128, device=cuda), x, 128, 100)
    h = torch.zeros(128, 128, device=cuda, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="T is not supported"):
        capi.transpose_aligned_128(torch.zeros_like(h), h, 128, 128)
