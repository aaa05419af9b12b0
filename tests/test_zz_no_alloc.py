"""The entry point for callers that cannot allocate device memory
(llmmm_fp8_blockwise_mm_e4m3out_noalloc): same kernel as the decode path of
llmmm_fp8_blockwise_mm_e4m3out, but its split-K scratch is an array inside the
library instead of a caller-owned workspace.  Both entry points must therefore
agree bit for bit (this path is integer/byte output with IEEE-derived scales;
the other FP8 tests use no looser tolerance for kernel-vs-kernel comparisons),
on two calls in a row, since the second call meets the scratch the first one
left behind.  The shapes are chosen so that most of them really take the
stream-K kernel (the one that exchanges partial tiles through the built-in
array) rather than the cluster kernel, which needs no scratch;
the test asserts which one runs.  Collected last on purpose (file name), runs
alone as well."""
import numpy as np
import pytest
import torch

from helpers import fp8_sources

pytestmark = pytest.mark.gpu


def make_inputs(oracle, cuda, seed, M, N, K):
    x, w = fp8_sources(seed, M, N, K, w_std=0.02)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    return [torch.from_numpy(a).to(cuda) for a in (A_q, A_s, B_q, B_s)]


# (M, N, K, kernel the launch heuristics must pick).  Order matters: the wide gate_up shape runs first and leaves
# the scratch behind (all zero again, if the readers cleared what they consumed) for the narrower ones that follow.
SHAPES = [
    (1, 19456, 2560, "stream-K"),   # 152 output groups: more than the SMs, no cluster size fits
    (16, 1280, 4096, "stream-K"),   # 10 groups: clusters of 7 would leave half of the SMs idle
    (4, 384, 4096, "stream-K"),     # 96 weight blocks on 96 CTAs: 32 contributors per output group
    (13, 19456, 2560, "stream-K"),  # ragged M
    (1, 2560, 4096, "cluster"),     # takes no scratch at all
    (16, 6144, 2560, "cluster"),
    (5, 384, 128, "stream-K"),      # one K-block: every segment is whole, nothing is published
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_noalloc_matches_workspace_entry_point_twice(capi, oracle, cuda, shape):
    M, N, K, kernel = shape
    first = make_inputs(oracle, cuda, 90, M, N, K)
    second = make_inputs(oracle, cuda, 91, M, N, K)
    capi.ensure_workspace(M, N, K)
    # both entry points make the same choice between the cluster and the stream-K kernel; the plan text of the
    # regular entry (with its workspace registered) names it
    assert kernel in capi.describe_plan("fp8", M, N, K)
    for A_q, A_s, B_q, B_s in (first, second):
        ref_q = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
        ref_s = torch.full((N // 128, M), float("nan"), device=cuda)
        got_q = torch.full((M, N), 0x55, dtype=torch.uint8, device=cuda)
        got_s = torch.full((N // 128, M), float("nan"), device=cuda)
        capi.fp8_blockwise_mm(A_q, A_s, B_q, B_s, ref_q, ref_s, M, N, K)
        capi.fp8_blockwise_mm_noalloc(A_q, A_s, B_q, B_s, got_q, got_s, M, N, K)
        torch.cuda.synchronize()
        capi.check_status()
        assert torch.equal(got_s, ref_s)
        assert torch.equal(got_q, ref_q)
    # and the result is the right one, not merely the same one
    A_q, A_s, B_q, B_s = (t.cpu().numpy() for t in second)
    o_q, o_s, _ = oracle.fp8_blockwise_mm(A_q, A_s, B_q, B_s)
    assert np.abs(got_s.cpu().numpy() / o_s - 1).max() <= 4e-6
    assert (got_q.cpu().numpy() == o_q).mean() > 0.99


def test_noalloc_rejects_sizes_beyond_its_scratch(capi, cuda):
    z8 = torch.zeros(17, 256, dtype=torch.uint8, device=cuda)
    zs = torch.zeros(2, 17, device=cuda)
    w8 = torch.zeros(256, 256, dtype=torch.uint8, device=cuda)
    ws = torch.zeros(2, 2, device=cuda)
    with pytest.raises(RuntimeError, match="M <= 16"):
        capi.fp8_blockwise_mm_noalloc(z8, zs, w8, ws, z8, zs, 17, 256, 256)
    with pytest.raises(RuntimeError, match="not aligned"):
        capi.fp8_blockwise_mm_noalloc(z8, zs, w8, ws, z8, zs, 16, 200, 256)
