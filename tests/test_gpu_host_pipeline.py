"""The host-buffer entry (copy in, GEMM, copy out, successive calls overlapped) returns, for every call, exactly
what the device-resident C ABI call returns for the same operands."""
import numpy as np
import pytest
import torch

from llmmm_b200.host_pipeline import Fp8GemmHostPipeline
from test_gpu_fp8 import check_against_oracle, make_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(384, 640, 1024), (16, 2560, 4096)])
def test_pipeline_matches_direct_calls(capi, oracle, cuda, shape):
    M, N, K = shape
    cases = [make_case(oracle, 70 + i, M, N, K) for i in range(5)]  # more calls than pipeline slots
    pipe = Fp8GemmHostPipeline(M, N, K, depth=2, device=cuda)
    host_in = [[torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in case] for case in cases]
    host_out = [(torch.empty(M, N, dtype=torch.uint8).pin_memory(), torch.empty(N // 128, M).pin_memory())
                for _ in cases]
    for hin, hout in zip(host_in, host_out):
        pipe.submit(*hin, *hout)
    pipe.drain()
    assert pipe.calls == 5
    for case, hin, (hq, hs) in zip(cases, host_in, host_out):
        dA, dAs, dB, dBs = (t.to(cuda) for t in hin)
        Cq = torch.empty(M, N, dtype=torch.uint8, device=cuda)
        Cs = torch.empty(N // 128, M, device=cuda)
        Cf = torch.empty(M, N, device=cuda)
        capi.fp8_blockwise_mm(dA, dAs, dB, dBs, Cq, Cs, M, N, K)
        capi.fp8_blockwise_mm_f32(dA, dAs, dB, dBs, Cf, M, N, K)
        torch.cuda.synchronize()
        assert torch.equal(hq, Cq.cpu()) and torch.equal(hs, Cs.cpu())
        check_against_oracle(oracle, *case, hq.numpy(), hs.numpy(), Cf.cpu().numpy())
    capi.check_status()


def test_pipeline_rejects_misaligned_shapes(cuda):
    with pytest.raises(RuntimeError, match="not aligned"):
        Fp8GemmHostPipeline(128, 100, 128, device=cuda)
