"""llmmm_describe_plan / llmmm_tune: the launch heuristics as text, and the warm-up that the reference's planned
functor calls tune(N, K) (src/mm/fp32/impl.h:20).  The descriptions are checked against the behaviour they
describe (split launches counted, decode path taken)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tune_then_first_call_and_descriptions(capi, cuda):
    for kind in ("fp16", "bf16", "fp8", "fp8_f32out"):
        capi.tune(kind, 4096, 4096)
    capi.clear_workspace()
    assert "fp16_gemm_kernel<__half>" in capi.describe_plan("fp16", 128, 4096, 4096)
    d = capi.describe_plan("bf16", 4096, 4096, 4096)
    assert "fp16_gemm_pair_kernel<__nv_bfloat16>" in d and "256 tiles" in d and "no split" in d
    d = capi.describe_plan("fp8", 4096, 4096, 4096)
    assert "fp8_blockwise_gemm_pair_kernel<false>" in d and "no split" in d
    assert "fp8_blockwise_gemm_kernel<true>" in capi.describe_plan("fp8_f32out", 100, 4096, 4096)
    # M <= 64 without scratch: cluster path where clusters fill the GPU, otherwise the general kernel
    assert "cluster" in capi.describe_plan("fp8", 1, 6144, 2560)
    assert "fp8_blockwise_gemm_kernel<false>" in capi.describe_plan("fp8", 64, 19456, 2560)
    # with scratch registered the same questions get the split answers, and launches agree with them
    capi.ensure_workspace(4096, 4096, 4096)
    capi.ensure_workspace(64, 19456, 2560)
    d = capi.describe_plan("fp8", 4096, 4096, 4096)
    assert "34 tiles cut 2-way along K" in d and "222 whole tiles" in d
    assert "stream-K" in capi.describe_plan("fp8", 64, 19456, 2560)
    n0 = capi.split_launch_count()
    capi.describe_plan("fp16", 4096, 4096, 4096)
    assert capi.split_launch_count() == n0  # a question is not a launch
    A = torch.zeros(4096, 4096, dtype=torch.uint8, device=cuda)
    S = torch.ones(32, 4096, device=cuda)
    Bs = torch.ones(32, 32, device=cuda)
    C = torch.empty(4096, 4096, dtype=torch.uint8, device=cuda)
    Cs = torch.empty(32, 4096, device=cuda)
    capi.fp8_blockwise_mm(A, S, A, Bs, C, Cs, 4096, 4096, 4096)
    torch.cuda.synchronize()
    assert capi.split_launch_count() == n0 + 1
    capi.check_status()
