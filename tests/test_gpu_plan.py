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


def _time_decode(capi, cuda, M, N, K, copies=24, reps=5):
    """Median microseconds per launch over weight copies that together exceed L2.  The launches are replayed from
    a CUDA graph: issued one by one from Python these kernels (5-10 us) would be timed by the host's launch path,
    which differs between a cluster launch and a plain one, not by the GPU."""
    xq = torch.randint(0, 120, (M, K), dtype=torch.uint8, device=cuda)
    xs = torch.rand(K // 128, M, device=cuda)
    ws = [(torch.randint(0, 120, (N, K), dtype=torch.uint8, device=cuda), torch.rand(N // 128, K // 128, device=cuda))
          for _ in range(copies)]
    cq = torch.empty(M, N, dtype=torch.uint8, device=cuda)
    cs = torch.empty(N // 128, M, device=cuda)

    def chain():
        for w in ws:
            capi.fp8_blockwise_mm(xq, xs, w[0], w[1], cq, cs, M, N, K)

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    times = []
    with torch.cuda.stream(stream):
        chain()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            chain()
        for _ in range(reps + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / copies)
    torch.cuda.current_stream().wait_stream(stream)
    return sorted(times[1:])[len(times[1:]) // 2], cq, cs


def test_tune_measures_the_decode_plans(capi, cuda):
    """llmmm_tune(fp8, N, K) times stream-K and every cluster size that fits for M = 16 / 32 / 64 and records
    the winner: afterwards the plan text says so, the tuned call is not slower than the default rule's choice
    was, and the result is the same bytes (every plan adds the partial sums of a K-block range in a fixed order;
    the ranges differ between plans, so scales may differ in the last bit: compared through the de-quantised
    values)."""
    N, K = 2560, 4096
    capi.ensure_workspace(64, N, K)
    capi.ensure_workspace(4096, N, K)  # the pair kernel's split scratch: the 65..128-row choice is measured with it
    before = {}
    for M in (16, 64):
        assert "default rule" in capi.describe_plan("fp8", M, N, K)
        before[M] = _time_decode(capi, cuda, M, N, K)
    capi.tune("fp8", N, K)
    for M in (16, 64):
        assert "measured by llmmm_tune" in capi.describe_plan("fp8", M, N, K)
        us, cq, cs = _time_decode(capi, cuda, M, N, K)
        assert us <= before[M][0] * 1.10, (M, us, before[M][0])
    capi.check_status()
    # the same call also measured the single-CTA kernel against the pair kernel for 65..128 rows of this weight
    assert "kernel choice: measured by llmmm_tune" in capi.describe_plan("fp8", 128, N, K)
    assert "kernel choice: default rule" in capi.describe_plan("fp8", 128, 6144, 2560)
    # a shape the tuner has not seen keeps the default rule
    assert "default rule" in capi.describe_plan("fp8", 16, 6144, 2560)
