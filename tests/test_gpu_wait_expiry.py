"""Failure detection without a fault: a kernel whose wait can never be satisfied gives up after its limit,
ends normally, and the host reads the reason from the status word; the context stays usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_is_reported(capi, cuda):
    L = capi.lib()
    capi.check_status()  # clean slate
    assert L.llmmm_selftest_wait_expiry(2000, None) == 0  # 2 ms limit
    with pytest.raises(RuntimeError, match="0x1ff"):
        capi.check_status()
    capi.check_status()  # the word was cleared by the read
    # the context is intact: a normal GEMM still runs and is right
    A = torch.eye(256, device=cuda, dtype=torch.float16)
    B = torch.rand(256, 256, device=cuda).half()
    C = torch.zeros(256, 256, device=cuda, dtype=torch.float16)
    capi.fp16_mm(A, B, C, 256, 256, 256)
    assert torch.equal(C, B)
    capi.check_status()


def test_selftest_argument_check(capi, cuda):
    assert capi.lib().llmmm_selftest_wait_expiry(0, None) == 1
