"""Explicit-workspace entry points (llmmm_*_ws): the split-K scratch is an argument of the call.  Two streams with
two buffers run the same split problems at the same time; each result must be bit-equal to the run that was
alone on the device (the sums of a split are taken in a fixed order), and nothing may depend on the buffer
registered for the device -- there is none in this test."""
import pytest
import torch

from test_gpu_fp8 import full_size_case

pytestmark = pytest.mark.gpu


def _problem(capi, cuda, M, N, K, seed):
    A_q, A_s, B_q, B_s = full_size_case(capi, cuda, M, N, K, seed, 0.02)
    return A_q, A_s, B_q, B_s


@pytest.mark.parametrize("shape", [(16, 19456, 2560), (64, 2560, 9728), (4096, 4096, 4096)],
                         ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_two_streams_two_buffers_match_serial_runs(capi, cuda, shape):
    M, N, K = shape
    capi.clear_workspace()  # nothing registered: the explicit buffers are all the scratch there is
    need = max(capi.fp8_workspace_bytes(M, N, K), capi.fp8_workspace_bytes(4096, 4096, 4096))
    probs = [_problem(capi, cuda, M, N, K, 80 + i) for i in range(2)]
    bufs = [torch.empty(need, dtype=torch.uint8, device=cuda).fill_(0x5a) for _ in range(2)]
    streams = [torch.cuda.Stream(device=cuda) for _ in range(2)]
    torch.cuda.synchronize()
    for b, s in zip(bufs, streams):
        capi.prepare_workspace(b, stream=s)
    split0 = capi.split_launch_count()

    def run(i, stream):
        Cq = torch.full((M, N), 0xAA, dtype=torch.uint8, device=cuda)
        Cs = torch.full((N // 128, M), float("nan"), device=cuda)
        capi.fp8_blockwise_mm_ws(*probs[i], Cq, Cs, M, N, K, bufs[i], stream=stream)
        return Cq, Cs

    # serial: one at a time
    serial = []
    for i in range(2):
        serial.append(run(i, streams[i]))
        torch.cuda.synchronize()
    # concurrent: many launches in flight on both streams
    for _ in range(3):
        outs = [[], []]
        for _rep in range(6):
            for i in range(2):
                with torch.cuda.stream(streams[i]):
                    outs[i].append(run(i, streams[i]))
        torch.cuda.synchronize()
        capi.check_status()
        for i in range(2):
            for Cq, Cs in outs[i]:
                assert torch.equal(Cq, serial[i][0]) and torch.equal(Cs, serial[i][1])
    if M > 128:
        assert capi.split_launch_count() > split0  # the buffers were really used: the last wave was cut along K
    else:
        assert "stream-K" in _plan_with(capi, bufs[0], M, N, K) or "cluster" in _plan_with(capi, bufs[0], M, N, K)
    # the same call without scratch still computes (unsplit), and gives the same bytes up to the order of fp32 sums
    Cq = torch.empty(M, N, dtype=torch.uint8, device=cuda)
    Cs = torch.empty(N // 128, M, device=cuda)
    capi.fp8_blockwise_mm_ws(*probs[0], Cq, Cs, M, N, K, None)
    torch.cuda.synchronize()
    capi.check_status()
    assert (Cq == serial[0][0]).float().mean().item() > 0.99


def _plan_with(capi, buf, M, N, K):
    from llmmm_b200.capi import lib, _check
    _check(lib().llmmm_bind_workspace(buf.data_ptr(), buf.numel()))
    try:
        return capi.describe_plan("fp8", M, N, K)
    finally:
        _check(lib().llmmm_bind_workspace(None, 0))


def test_ws_argument_errors(capi, cuda):
    z8 = torch.zeros(128 * 128, dtype=torch.uint8, device=cuda)
    zf = torch.zeros(128 * 128, dtype=torch.float32, device=cuda)
    small = torch.zeros(1024, dtype=torch.uint8, device=cuda)
    with pytest.raises(RuntimeError, match="workspace must be 256-byte aligned"):
        capi.fp8_blockwise_mm_ws(z8, zf, z8, zf, z8, zf, 128, 128, 128, small)
    with pytest.raises(RuntimeError, match="workspace must be 256-byte aligned"):
        capi.prepare_workspace(small)
