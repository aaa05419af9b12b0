"""Every element of the full-size outputs against a GPU-side fp64 reference (tests/gpu_reference.py, the
reference's double-accumulator test GEMM, test/kahan.cu:39-56, for quantised operands).  The reference's own
FP16 test compares the whole 4096^2 output the same way (test/fp16_mm_test.cc:31-36, 63-82).  Shapes: 4096^3,
the four Qwen3-4B linears at M = 4096, both 7B-scale MLP GEMMs at M = 8192 and one column shard of each per
world size of an N-split (2, 4, 8 ranks; the 28-group down projection splits unevenly over 8), all with the
split-K scratch registered.

Gates (the ones of tests/test_gpu_fp8.py, applied to every element):
  * fp32 accumulator within 4e-6 * row-amax of the fp64 ground truth;
  * fused C_q / C_s bit-exactly the quantisation rule applied to the kernel's own accumulator;
  * de-quantised C within half an e4m3 ulp (times the scale) of the accumulator it was rounded from, plus the
    accumulator tolerance above -- which is at most the oracle's own error + 1 ulp, the north-star gate."""
import numpy as np
import pytest
import torch

import gpu_reference as ref
from test_gpu_fp8 import full_size_case, gpu_c_quant, make_case

pytestmark = pytest.mark.gpu


def test_gpu_reference_matches_cpu_oracle(oracle, cuda):
    """Pins the GPU checker itself: equal to oracle.fp8_blockwise_acc(exact=True) to fp64 rounding."""
    for (M, N, K) in [(37, 256, 384), (128, 384, 1024)]:
        A_q, A_s, B_q, B_s = make_case(oracle, 70, M, N, K)
        t0 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True)
        dev = [torch.from_numpy(np.ascontiguousarray(a)).to(cuda) for a in (A_q, A_s, B_q, B_s)]
        got = ref.fp8_blockwise_acc_f64(*dev).cpu().numpy()
        assert np.abs(got - t0).max() <= 1e-13 * np.abs(t0).max()
        part = ref.fp8_blockwise_acc_f64(*dev, col0=128, cols=128).cpu().numpy()
        assert np.array_equal(part, got[:, 128:256])


def check_every_element(capi, cuda, A_q, A_s, B_q, B_s, t0):
    M, K = A_q.shape
    N = B_q.shape[0]
    Cq = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
    Cs = torch.full((N // 128, M), float("nan"), device=cuda)
    Cf = torch.full((M, N), float("nan"), device=cuda)
    capi.fp8_blockwise_mm(A_q, A_s, B_q, B_s, Cq, Cs, M, N, K)
    capi.fp8_blockwise_mm_f32(A_q, A_s, B_q, B_s, Cf, M, N, K)
    torch.cuda.synchronize()
    capi.check_status()
    tol = 4e-6 * t0.abs().amax(dim=1, keepdim=True)
    # 1. the accumulator, every element
    err = (Cf.double() - t0).abs()
    assert bool((err <= tol).all()), float((err / tol).max())
    # 2. fused output == rule(own accumulator), bit for bit
    q_rule, s_rule = gpu_c_quant(Cf)
    assert torch.equal(Cs, s_rule) and torch.equal(Cq, q_rule)
    # 3. de-quantised output against the ground truth
    scale = Cs.t().repeat_interleave(128, dim=1).double()
    deq = ref.e4m3_table(cuda)[Cq.long()] * scale
    bound = 0.5 * ref.e4m3_ulp(Cq) * scale * (1 + 1e-6) + tol
    assert bool(((deq - t0).abs() <= bound).all())


@pytest.mark.parametrize("shape", [(4096, 4096, 4096, 1.0), (4096, 6144, 2560, 0.02), (4096, 2560, 4096, 0.02),
                                   (4096, 19456, 2560, 0.02), (4096, 2560, 9728, 0.02)],
                         ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_every_element_prefill_shapes(capi, cuda, shape):
    M, N, K, w_std = shape
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, 61, w_std)
    capi.ensure_workspace(M, N, K)
    check_every_element(capi, cuda, A_q, A_s, B_q, B_s, ref.fp8_blockwise_acc_f64(A_q, A_s, B_q, B_s))


@pytest.mark.parametrize("NK", [(37888, 3584), (3584, 18944)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_every_element_7b_mlp_and_its_column_shards(capi, cuda, NK):
    from llmmm_b200 import shard
    M = 8192
    N, K = NK
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, 62, 0.02)
    capi.ensure_workspace(M, N, K)
    t0 = ref.fp8_blockwise_acc_f64(A_q, A_s, B_q, B_s)
    check_every_element(capi, cuda, A_q, A_s, B_q, B_s, t0)
    # one column shard per world size, the last rank's (the short one where the groups do not divide evenly)
    for world in (2, 4, 8):
        n0, n1 = shard.split_n(N, world, world - 1)
        Bq_r = B_q[n0:n1].contiguous()
        Bs_r = B_s[n0 // 128:n1 // 128].contiguous()
        check_every_element(capi, cuda, A_q, A_s, Bq_r, Bs_r, t0[:, n0:n1])
