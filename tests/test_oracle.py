"""CPU tests of the oracle itself: codec known answers, agreement between its
tiers, and the algebraic properties the reference's quantisation rules imply."""
import numpy as np
import pytest

from helpers import fp16_inputs, fp8_sources


def test_e4m3_known_answers(oracle):
    # values probed from the CUDA toolkit's own host conversion (cuda_fp8.h)
    x = np.array([0.0, 448.0, 449.0, 1e9, -1e9, 17.5, 2.0 ** -9, 2.0 ** -10, 1.0, -1.0, 0.875, 464.1], np.float32)
    q = oracle.e4m3_encode(x)
    back = oracle.e4m3_decode(q)
    assert back.tolist() == [0.0, 448.0, 448.0, 448.0, -448.0, 18.0, 2.0 ** -9, 0.0, 1.0, -1.0, 0.875, 448.0]
    assert q[1] == 0x7E and q[4] == 0xFE and q[8] == 0x38


def test_e4m3_roundtrip_all_codes(oracle):
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)  # skip NaN
    vals = oracle.e4m3_decode(codes)
    again = oracle.e4m3_encode(vals)
    # -0 re-encodes to 0x80
    assert (again == codes).all()
    assert np.abs(vals).max() == 448.0


def test_e4m3_round_to_nearest_even(oracle):
    # halfway between 16 (0x58) and 18 (0x59) is 17 -> even mantissa (16); between 18 and 20 is 19 -> 20
    q = oracle.e4m3_decode(oracle.e4m3_encode(np.array([17.0, 19.0, 17.0001, 18.9999], np.float32)))
    assert q.tolist() == [16.0, 20.0, 18.0, 18.0]


def test_f16_bf16_codecs(oracle):
    x = np.array([1.0, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, 65504.0, 1e-8, -0.333], np.float32)
    assert (oracle.to_f16_bits(x) == x.astype(np.float16).view(np.uint16)).all()
    b = oracle.from_bf16_bits(oracle.to_bf16_bits(x))
    assert np.allclose(b, x, rtol=2.0 ** -8)
    assert oracle.to_bf16_bits(np.array([1.0 + 2.0 ** -8], np.float32))[0] == 0x3F80  # tie -> even


def test_reference_gemms_agree(oracle):
    A, B = fp16_inputs(1, 64, 96, 512)
    exact = oracle.exact_gemm(A, B)
    kahan = oracle.kahan_gemm(A, B)
    dbl = oracle.double_gemm(A, B)
    # Kahan keeps the error at a few ulps of the result whatever K is
    assert np.abs(kahan - exact).max() <= 4 * np.finfo(np.float32).eps * np.abs(exact).max()
    # the double version rounds each product to fp32 first: error ~ K * eps/2 * |a*b|
    assert np.abs(dbl - exact).max() <= 512 * np.finfo(np.float32).eps
    # a slab equals the matching rows of the whole
    assert (oracle.kahan_gemm(A, B, 16, 8) == kahan[16:24]).all()


def test_kahan_beats_naive_sum(oracle):
    rng = np.random.default_rng(5)
    A = rng.uniform(0.5, 1.0, (4, 8192)).astype(np.float32)
    B = rng.uniform(0.5, 1.0, (8192, 8)).astype(np.float32)
    exact = oracle.exact_gemm(A, B)
    naive = np.zeros((4, 8), np.float32)
    for k in range(8192):
        naive += A[:, k:k + 1] * B[k:k + 1, :]
    assert np.abs(oracle.kahan_gemm(A, B) - exact).max() < 0.05 * np.abs(naive - exact).max()


def test_quant_1x128_rules(oracle):
    x, _ = fp8_sources(2, 40, 128, 384)
    x[7, 128:256] = 0.0
    q, s = oracle.quant_1x128(x)
    assert q.shape == (40, 384) and s.shape == (3, 40)
    amax = np.abs(x.reshape(40, 3, 128)).max(axis=2)
    assert (s.T == (amax / np.float32(448.0)).astype(np.float32)).all()
    deq = oracle.e4m3_decode(q)
    # the element that attains amax maps to +-448 exactly; an all-zero group gives scale 0 and zeros
    assert (np.abs(deq.reshape(40, 3, 128)).max(axis=2)[amax > 0] == 448.0).all()
    assert s[1, 7] == 0.0 and (q[7, 128:256] == 0).all()
    # de-quantisation error is at most half an e4m3 ulp of 448 (=16) times the scale
    err = np.abs(deq * np.repeat(s.T, 128, axis=1) - x)
    assert (err <= 16.0 * np.repeat(s.T, 128, axis=1) * 1.0001 + 1e-12).all()


def test_quant_128x128_rules(oracle):
    _, w = fp8_sources(3, 8, 256, 384, w_std=0.02)
    q, s = oracle.quant_128x128(w)
    assert s.shape == (2, 3)
    amax = np.abs(w.reshape(2, 128, 3, 128)).max(axis=(1, 3))
    assert (s == (amax / np.float32(448.0)).astype(np.float32)).all()
    # quantising a block on its own gives the same bytes as quantising it inside the matrix
    q11, s11 = oracle.quant_128x128(w[128:256, 128:256])
    assert (q11 == q[128:256, 128:256]).all() and s11[0, 0] == s[1, 1]


def test_blockwise_gemm_tiers(oracle):
    x, w = fp8_sources(4, 48, 256, 512, w_std=0.02)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    t1 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s)
    t0 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True)
    assert np.abs(t1 - t0).max() <= 2e-6 * np.abs(t0).max()
    # independent restatement with numpy in float64
    a = oracle.e4m3_decode(A_q).astype(np.float64) * np.repeat(A_s.T.astype(np.float64), 128, axis=1)
    b = oracle.e4m3_decode(B_q).astype(np.float64) * np.kron(B_s.astype(np.float64), np.ones((128, 128)))
    assert np.abs(a @ b.T - t0).max() <= 1e-6 * np.abs(t0).max()
    # row slabs agree with the whole
    assert (oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s, row0=8, rows=5) == t1[8:13]).all()
    # quantisation noise of the operands stays small against the fp32 product
    assert np.abs(x.astype(np.float64) @ w.T.astype(np.float64) - t0).max() <= 0.1 * np.abs(t0).max()


def test_c_quant_rules(oracle):
    rng = np.random.default_rng(6)
    acc = rng.standard_normal((20, 256)).astype(np.float32) * 3
    acc[5, :128] = 0.0
    q, s = oracle.c_quant_1x128(acc)
    amax = np.abs(acc.reshape(20, 2, 128)).max(axis=2)
    assert (s.T == (amax / np.float32(448.0)).astype(np.float32)).all()
    assert s[0, 5] == 0.0 and (q[5, :128] == 0).all()  # the defined all-zero case
    deq = oracle.dequant_1x128(q, s)
    assert (np.abs(deq - acc) <= 16.0 * np.repeat(s.T, 128, axis=1) * 1.001 + 1e-12).all()
    # idempotence: quantising the de-quantised values reproduces the same bytes
    q2, s2 = oracle.c_quant_1x128(deq)
    assert (q2 == q).all()
    assert np.allclose(s2, s, rtol=1e-6)


def test_linearity_of_blockwise_gemm(oracle):
    # scaling the activation scales by a power of two scales the accumulator exactly
    x, w = fp8_sources(7, 16, 128, 256, w_std=0.02)
    A_q, A_s = oracle.quant_1x128(x)
    B_q, B_s = oracle.quant_128x128(w)
    t1 = oracle.fp8_blockwise_acc(A_q, A_s, B_q, B_s)
    t1x4 = oracle.fp8_blockwise_acc(A_q, A_s * np.float32(4.0), B_q, B_s)
    assert (t1x4 == t1 * np.float32(4.0)).all()
    cq, cs = oracle.c_quant_1x128(t1)
    cq4, cs4 = oracle.c_quant_1x128(t1x4)
    assert (cq == cq4).all() and (cs4 == cs * np.float32(4.0)).all()


def test_transpose(oracle):
    rng = np.random.default_rng(8)
    a = rng.integers(0, 255, (128, 256), dtype=np.uint8)
    f = rng.standard_normal((128, 256)).astype(np.float32)
    assert (oracle.transpose(a) == a.T).all() and (oracle.transpose(f) == f.T).all()


def test_qk_norm_rope_against_torch(oracle):
    # the hook's restatement against an independent torch formulation (rotate-half rotary embedding, RMSNorm
    # over the head), in fp64; properties: value heads untouched, the rotation keeps each head's norm
    import torch
    rng = np.random.default_rng(3)
    M, n_q, n_kv = 5, 3, 2
    acc = rng.standard_normal((M, (n_q + 2 * n_kv) * 128))
    pos = np.array([0, 7, 3, 100, 7], np.int32)
    ang = np.arange(128, dtype=np.float64)[:, None] / (1e4 ** (np.arange(64) / 64))[None, :]
    cos, sin = np.cos(ang), np.sin(ang)
    q_w, k_w = 1 + 0.1 * rng.standard_normal(128), 1 + 0.1 * rng.standard_normal(128)
    got = oracle.qk_norm_rope(acc, pos, cos, sin, q_w, k_w, 1e-6, n_q, n_kv)

    x = torch.from_numpy(acc).view(M, n_q + 2 * n_kv, 128)
    c = torch.from_numpy(np.concatenate([cos, cos], 1))[torch.from_numpy(pos).long()][:, None, :]
    s = torch.from_numpy(np.concatenate([sin, sin], 1))[torch.from_numpy(pos).long()][:, None, :]

    def hook(h, w):
        h = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + 1e-6) * torch.from_numpy(w)
        rot = torch.cat([-h[..., 64:], h[..., :64]], -1)
        return h * c + rot * s

    want = torch.cat([hook(x[:, :n_q], q_w), hook(x[:, n_q:n_q + n_kv], k_w), x[:, n_q + n_kv:]], 1).reshape(M, -1).numpy()
    assert np.abs(got - want).max() < 1e-12
    assert (got[:, (n_q + n_kv) * 128:] == acc[:, (n_q + n_kv) * 128:]).all()
    plain = oracle.qk_norm_rope(acc, pos, cos, sin, None, None, 1e-6, n_q, n_kv)
    n0 = np.linalg.norm(acc.reshape(M, -1, 128), axis=2)
    assert np.abs(np.linalg.norm(plain.reshape(M, -1, 128), axis=2) - n0).max() < 1e-12
    # the fp32 form stays within fp32 rounding of the fp64 one
    got32 = oracle.qk_norm_rope(acc.astype(np.float32), pos, cos.astype(np.float32), sin.astype(np.float32),
                                q_w.astype(np.float32), k_w.astype(np.float32), 1e-6, n_q, n_kv)
    assert got32.dtype == np.float32 and np.abs(got32 - got).max() < 5e-6
