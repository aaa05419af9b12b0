"""Sharded execution on one GPU: the N-split and M-split shards of a GEMM, run one after the other through the
C ABI, must reproduce the unsharded run bit for bit (the path has no reduction) as long as no tile is cut along
K, i.e. without registered scratch.  With scratch a shard and the full problem may cut different tiles, so
there the results agree to the association of fp32 sums (scales within 4e-6, bytes almost all equal).  Shapes follow the 7B-scale
MLP configuration (hidden 3584, gate_up N=37888, down K=18944) at a reduced M so that the oracle can check
sampled rows; 37888 = 296 groups splits evenly over 8 ranks, 3584 = 28 groups does not (4,4,4,4,3,3,3,3)."""
import numpy as np
import pytest
import torch

from llmmm_b200 import shard
from test_gpu_fp8 import check_against_oracle, full_size_case

pytestmark = pytest.mark.gpu


def run(capi, cuda, A_q, A_s, B_q, B_s, scratch=False):
    M, K = A_q.shape
    N = B_q.shape[0]
    if scratch:
        capi.ensure_workspace(M, N, K)
    else:
        capi.clear_workspace()
    Cq = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
    Cs = torch.full((N // 128, M), float("nan"), device=cuda)
    capi.fp8_blockwise_mm(A_q, A_s, B_q.contiguous(), B_s.contiguous(), Cq, Cs, M, N, K)
    return Cq, Cs


@pytest.mark.parametrize("shape,world", [((256, 37888, 3584), 8), ((384, 3584, 18944), 8), ((512, 3584, 2048), 3)])
def test_n_split_is_bitwise_the_unsharded_result(capi, oracle, cuda, shape, world):
    M, N, K = shape
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, 95, 0.02)
    full_q, full_s = run(capi, cuda, A_q, A_s, B_q, B_s)
    for rank in range(world):
        n0, n1 = shard.split_n(N, world, rank)
        bq, bs = shard.shard_weights_n(B_q, B_s, world, rank)
        cq, cs = run(capi, cuda, A_q, A_s, bq, bs)
        assert torch.equal(cq, full_q[:, n0:n1])
        assert torch.equal(cs, full_s[n0 // 128:n1 // 128])
        if rank in (0, world - 1):
            sq, ss = run(capi, cuda, A_q, A_s, bq, bs, scratch=True)
            ref_s = full_s[n0 // 128:n1 // 128]
            assert bool(((ss - ref_s).abs() <= 4e-6 * ref_s.abs()).all())
            assert float((sq == full_q[:, n0:n1]).float().mean()) > 0.999
    torch.cuda.synchronize()
    capi.check_status()
    # and the unsharded result is right: sampled rows against the CPU oracle
    hA_q, hA_s, hB_q, hB_s = (t.cpu().numpy() for t in (A_q, A_s, B_q, B_s))
    Cf = torch.empty(M, N, device=cuda)
    capi.clear_workspace()  # the accumulator of the same, unsplit, schedule that produced full_q
    capi.fp8_blockwise_mm_f32(A_q, A_s, B_q, B_s, Cf, M, N, K)
    check_against_oracle(oracle, hA_q, hA_s, hB_q, hB_s, full_q.cpu().numpy(), full_s.cpu().numpy(), Cf.cpu().numpy(),
                         rows=(M - 2, 2))


@pytest.mark.parametrize("world", [2, 3])
def test_m_split_is_bitwise_the_unsharded_result(capi, cuda, world):
    M, N, K = 1000, 2560, 4096  # ragged row split; shards of 333/334 and 500 rows
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, 96, 0.02)
    full_q, full_s = run(capi, cuda, A_q, A_s, B_q, B_s)
    for rank in range(world):
        m0, m1 = shard.split_m(M, world, rank)
        aq, as_ = shard.shard_activations_m(A_q, A_s, world, rank)
        cq, cs = run(capi, cuda, aq, as_, B_q, B_s)
        assert torch.equal(cq, full_q[m0:m1])
        assert torch.equal(cs, full_s[:, m0:m1])
    capi.check_status()


@pytest.mark.parametrize("shape,world", [((384, 1536, 1024), 3), ((4096, 4096, 4096), 2)])
def test_gather_epilogue_fills_every_destination(capi, cuda, shape, world):
    """The fused all-gather, on one GPU: every shard's GEMM stores its columns into all `world` destinations (here
    `world` local buffers standing in for the peers' mapped ones); afterwards each destination is the unsharded
    result, bit for bit (no scratch registered, so no tile is cut along K)."""
    M, N, K = shape
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, 97, 0.02)
    capi.clear_workspace()
    full_q, full_s = run(capi, cuda, A_q, A_s, B_q, B_s)
    dst_q = [torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda) for _ in range(world)]
    dst_s = [torch.full((N // 128, M), float("nan"), device=cuda) for _ in range(world)]
    for rank in range(world):
        n0, n1 = shard.split_n(N, world, rank)
        bq, bs = shard.shard_weights_n(B_q, B_s, world, rank)
        capi.fp8_blockwise_mm_gather(A_q, A_s, bq.contiguous(), bs.contiguous(), dst_q, dst_s, N, n0, M, n1 - n0, K)
    torch.cuda.synchronize()
    capi.check_status()
    for q, s in zip(dst_q, dst_s):
        assert torch.equal(q, full_q) and torch.equal(s, full_s)
    with pytest.raises(RuntimeError, match="128-column boundaries"):
        capi.fp8_blockwise_mm_gather(A_q, A_s, B_q, B_s, dst_q, dst_s, N, 64, M, N, K)
    with pytest.raises(RuntimeError, match="destinations"):
        capi.fp8_blockwise_mm_gather(A_q, A_s, B_q, B_s, [], [], N, 0, M, N, K)


def test_gather_epilogue_with_split_tiles(capi, cuda):
    """With scratch registered a shard's last wave is cut along K; the gather epilogue must then store exactly what
    the plain entry point stores for the same shard (same plan, same order of sums), at the shard's columns."""
    M, N, K, world = 512, 2048, 4096, 2
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, 98, 0.02)
    dst_q = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
    dst_s = torch.full((N // 128, M), float("nan"), device=cuda)
    n_split = capi.split_launch_count()
    for rank in range(world):
        n0, n1 = shard.split_n(N, world, rank)
        bq, bs = shard.shard_weights_n(B_q, B_s, world, rank)
        bq, bs = bq.contiguous(), bs.contiguous()
        ref_q, ref_s = run(capi, cuda, A_q, A_s, bq, bs, scratch=True)
        capi.fp8_blockwise_mm_gather(A_q, A_s, bq, bs, [dst_q], [dst_s], N, n0, M, n1 - n0, K)
        torch.cuda.synchronize()
        assert torch.equal(dst_q[:, n0:n1], ref_q) and torch.equal(dst_s[n0 // 128:n1 // 128], ref_s)
    assert capi.split_launch_count() == n_split + 2 * world  # every one of these launches was split
    capi.check_status()
