"""Side-by-side run with the reference's own kernels (oracle/_ref, the
unmodified reference sources built for sm_100a): our outputs against theirs on
the same device buffers.  This is the "reference kernel error" tier of the FP8
tolerance, measured live instead of through the committed golden vectors."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import fp8_sources, fp16_inputs

pytestmark = pytest.mark.gpu

REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libllmmm_ref.so"
_vp = ctypes.c_void_p


@pytest.fixture(scope="module")
def ref():
    if not REF.exists():
        pytest.skip("oracle/_ref was not built (needs the reference checkout at build time)")
    return ctypes.CDLL(str(REF))


def test_fp16_against_reference_kernel(capi, oracle, cuda, ref):
    M = N = K = 512
    A, B = fp16_inputs(70, M, N, K)
    dA, dB = torch.from_numpy(A).to(cuda).half(), torch.from_numpy(B).to(cuda).half()
    ours = torch.zeros(M, N, device=cuda, dtype=torch.float16)
    theirs = torch.zeros(M, N, device=cuda, dtype=torch.float16)
    capi.fp16_mm(dA, dB, ours, M, N, K)
    assert ref.ref_fp16_mm_f16(_vp(dA.data_ptr()), _vp(dB.data_ptr()), _vp(theirs.data_ptr()), M, N, K, None) == 0
    torch.cuda.synchronize()
    exact = oracle.exact_gemm(dA.float().cpu().numpy(), dB.float().cpu().numpy())
    e_ours = np.abs(ours.float().cpu().numpy() - exact).max()
    e_ref = np.abs(theirs.float().cpu().numpy() - exact).max()
    assert e_ours <= e_ref * 1.5 + 1e-6
    assert (ours == theirs).float().mean().item() > 0.99


def test_fp8_against_reference_kernels(capi, oracle, cuda, ref):
    M, N, K = 256, 1024, 1024
    x, w = fp8_sources(71, M, N, K, w_std=0.02)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    t0 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True)
    dA, dAs, dB, dBs = (torch.from_numpy(a).to(cuda) for a in (A_q, A_s, B_q, B_s))
    Cq = torch.zeros(M, N, dtype=torch.uint8, device=cuda)
    Cs = torch.zeros(N // 128, M, device=cuda)
    capi.fp8_blockwise_mm(dA, dAs, dB, dBs, Cq, Cs, M, N, K)
    torch.cuda.synchronize()
    ours = oracle.dequant_1x128(Cq.cpu().numpy(), Cs.cpu().numpy())
    for name in ("ref_fp8_mm_opt_reg", "ref_fp8_mm_inner_split"):
        Rq = torch.zeros(M, N, dtype=torch.uint8, device=cuda)
        Rs = torch.zeros(N // 128, M, device=cuda)
        rc = getattr(ref, name)(_vp(dA.data_ptr()), _vp(dAs.data_ptr()), _vp(dB.data_ptr()), _vp(dBs.data_ptr()),
                                _vp(Rq.data_ptr()), _vp(Rs.data_ptr()), M, N, K, None)
        assert rc == 0
        torch.cuda.synchronize()
        theirs = oracle.dequant_1x128(Rq.cpu().numpy(), Rs.cpu().numpy())
        eps_ref = np.abs(theirs - t0).max()
        ulp_top = 32.0 * Cs.cpu().numpy().max()
        assert np.abs(ours - t0).max() <= eps_ref + ulp_top
        assert (Cq == Rq).float().mean().item() > 0.98
    # reference quantiser on the same buffer: identical bytes and scales
    dx = torch.from_numpy(x).to(cuda)
    q1 = torch.zeros(M, K, dtype=torch.uint8, device=cuda)
    s1 = torch.zeros(K // 128, M, device=cuda)
    q2, s2 = torch.zeros_like(q1), torch.zeros_like(s1)
    capi.fp8_quant_1x128(dx, q1, s1, M, K)
    ref.ref_fp8_quant_1x128(_vp(dx.data_ptr()), _vp(q2.data_ptr()), _vp(s2.data_ptr()), M, K, None)
    torch.cuda.synchronize()
    assert torch.equal(q1, q2) and torch.equal(s1, s2)
