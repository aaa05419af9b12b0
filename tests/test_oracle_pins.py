"""The oracle against golden vectors produced by the reference's OWN kernels
(built unmodified for sm_100a and run on a B200 by oracle/pin_against_ref.py;
outputs committed in tests/golden/ref_pins.npz).  Deterministic reference
kernels must match bit for bit; tensor-core kernels within their order-of-
summation noise."""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle.pin_against_ref import PIN_CASES, inputs_fp8, inputs_gemm

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def pins():
    return np.load(GOLD / "ref_pins.npz")


def test_summary_recorded_on_b200():
    s = json.loads((GOLD / "ref_pins.json").read_text())
    assert s["device"] == "NVIDIA B200"
    assert s["kahan_bit_exact"] and s["double_bit_exact"]
    assert s["quant_1x128_q_bit_exact"] and s["quant_1x128_scale_bit_exact"]
    assert s["cases"] == PIN_CASES


def test_kahan_and_double_gemm_bit_exact(oracle, pins):
    c = PIN_CASES["gemm"]
    A, B = inputs_gemm(c["seed"], c["M"], c["N"], c["K"])
    assert (oracle.kahan_gemm(A, B).view(np.uint32) == pins["kahan_C"].view(np.uint32)).all()
    assert (oracle.double_gemm(A, B).view(np.uint32) == pins["double_C"].view(np.uint32)).all()


def test_quant_1x128_bit_exact(oracle, pins):
    c = PIN_CASES["quant"]
    x = np.random.default_rng(c["seed"]).standard_normal((c["M"], c["K"])).astype(np.float32)
    x[3, 128:256] = 0.0
    q, s = oracle.quant_1x128(x)
    assert (q == pins["quant_q"]).all()
    assert (s.view(np.uint32) == pins["quant_s"].view(np.uint32)).all()


def test_fp16_reference_kernel_is_rounded_exact_product(oracle, pins):
    c = PIN_CASES["fp16"]
    A, B = inputs_gemm(c["seed"], c["M"], c["N"], c["K"])
    Ah, Bh = oracle.from_f16_bits(oracle.to_f16_bits(A)), oracle.from_f16_bits(oracle.to_f16_bits(B))
    exact = oracle.exact_gemm(Ah, Bh)
    ref = oracle.from_f16_bits(pins["fp16_C_bits"])
    # the reference kernel is the exact product rounded once, up to fp32 accumulation noise
    assert np.abs(ref - exact).max() <= 1e-3 * np.abs(exact).max()
    assert (oracle.to_f16_bits(exact.astype(np.float32)) == pins["fp16_C_bits"]).mean() > 0.99
    # and the Kahan reference GEMM agrees with the exact product to fp32 precision
    assert np.abs(oracle.kahan_gemm(Ah, Bh) - exact).max() <= 1e-5


def test_fp8_reference_kernel_matches_oracle(oracle, pins):
    c = PIN_CASES["fp8"]
    M, N, K = c["M"], c["N"], c["K"]
    x, w = inputs_fp8(c["seed"], M, N, K)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    q, s, acc = oracle.fp8_blockwise_mm(A_q, A_s, B_q, B_s)
    t0 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True)
    rq, rs = pins["fp8_mm_opt_reg_Cq"], pins["fp8_mm_opt_reg_Cs"]
    # scales: bit-identical for almost all groups, 1 ulp apart where the tensor core's summation
    # order moved the absmax, and a few groups where the reference kernel reports a LARGER scale
    # than its own rule amax/448 gives (never smaller, so nothing saturates)
    rel = rs / s
    assert (rs.view(np.uint32) == s.view(np.uint32)).mean() > 0.97
    assert rel.min() > 1 - 1e-6
    close = np.abs(rel - 1) < 1e-6
    assert close.mean() > 0.995
    # bytes: identical wherever the scale is identical, up to rounding ties moved by accumulation noise
    same_scale = np.repeat((rs.view(np.uint32) == s.view(np.uint32)).T, 128, axis=1)
    assert (rq == q)[same_scale].mean() > 0.999
    # de-quantised error against the fp64 ground truth: the oracle is as accurate as the reference kernel
    e_ref = np.abs(oracle.dequant_1x128(rq, rs) - t0).max()
    e_orc = np.abs(oracle.dequant_1x128(q, s) - t0).max()
    assert e_orc <= e_ref * 1.001
    # fp32-output kernel: the accumulator itself
    f32 = pins["fp8_mm_f32out_C_rows0_64"]
    assert np.abs(f32 - acc[:64]).max() <= 1e-6 * np.abs(acc).max()
