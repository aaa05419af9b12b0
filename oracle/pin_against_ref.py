"""Pins the CPU oracle against the reference's own kernels executed on a B200.

Needs a GPU and oracle/_ref/libllmmm_ref.so (the unmodified reference sources
built for sm_100a by `make -C oracle ref`).  For seeded inputs it runs the
reference's Kahan / double GEMMs, its 1x128 quantiser, its FP16 GEMM and its
FP8 fused-quant GEMM kernels, compares them with the oracle and writes

    <out>/ref_pins.npz   the reference kernels' outputs (golden vectors)
    <out>/ref_pins.json  the comparison summary

The committed copies live in tests/golden/; tests/test_oracle_pins.py re-checks
the oracle against them on any machine.  Usage (on a GPU box):

    python oracle/pin_against_ref.py --out <directory>
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from oracle import oracle as o  # noqa: E402

_vp = ctypes.c_void_p
_i = ctypes.c_int


def inputs_gemm(seed, M, N, K):
    rng = np.random.default_rng(seed)
    return (rng.uniform(-1, 1, (M, K)).astype(np.float32), rng.uniform(-1, 1, (K, N)).astype(np.float32))


def inputs_fp8(seed, M, N, K):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((M, K)).astype(np.float32), (rng.standard_normal((N, K)) * 0.02).astype(np.float32))


PIN_CASES = {
    "gemm": dict(seed=11, M=96, N=128, K=320),
    "quant": dict(seed=12, M=64, K=512),
    "fp16": dict(seed=13, M=256, N=256, K=256),
    "fp8": dict(seed=14, M=256, N=512, K=512),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="pins_out")
    args = ap.parse_args()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    R = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libllmmm_ref.so"))
    dev = torch.device("cuda:0")
    summary, arrays = {}, {}

    def d(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    # 1. reference GEMMs (test/kahan.cu)
    c = PIN_CASES["gemm"]
    A, B = inputs_gemm(c["seed"], c["M"], c["N"], c["K"])
    dA, dB = d(A), d(B)
    dC = torch.zeros(c["M"], c["N"], dtype=torch.float32, device=dev)
    R.ref_kahan(_vp(dA.data_ptr()), _vp(dB.data_ptr()), _vp(dC.data_ptr()), c["M"], c["N"], c["K"])
    ref_k = dC.cpu().numpy().copy()
    R.ref_fp32_naive_mm(_vp(dA.data_ptr()), _vp(dB.data_ptr()), _vp(dC.data_ptr()), c["M"], c["N"], c["K"])
    ref_d = dC.cpu().numpy().copy()
    summary["kahan_bit_exact"] = bool((o.kahan_gemm(A, B).view(np.uint32) == ref_k.view(np.uint32)).all())
    summary["double_bit_exact"] = bool((o.double_gemm(A, B).view(np.uint32) == ref_d.view(np.uint32)).all())
    arrays["kahan_C"], arrays["double_C"] = ref_k, ref_d

    # 2. activation quantiser <1,128,true>
    c = PIN_CASES["quant"]
    x = np.random.default_rng(c["seed"]).standard_normal((c["M"], c["K"])).astype(np.float32)
    x[3, 128:256] = 0.0  # an all-zero group exercises the s == 0 branch
    dx = d(x)
    dq = torch.zeros(c["M"], c["K"], dtype=torch.uint8, device=dev)
    ds = torch.zeros(c["K"] // 128, c["M"], dtype=torch.float32, device=dev)
    R.ref_fp8_quant_1x128(_vp(dx.data_ptr()), _vp(dq.data_ptr()), _vp(ds.data_ptr()), c["M"], c["K"], None)
    torch.cuda.synchronize()
    rq, rs = dq.cpu().numpy(), ds.cpu().numpy()
    oq, os_ = o.quant_1x128(x)
    summary["quant_1x128_q_bit_exact"] = bool((oq == rq).all())
    summary["quant_1x128_scale_bit_exact"] = bool((os_.view(np.uint32) == rs.view(np.uint32)).all())
    arrays["quant_q"], arrays["quant_s"] = rq, rs

    # 3. reference FP16 GEMM (src/mm/fp16)
    c = PIN_CASES["fp16"]
    A, B = inputs_gemm(c["seed"], c["M"], c["N"], c["K"])
    Ah, Bh = o.from_f16_bits(o.to_f16_bits(A)), o.from_f16_bits(o.to_f16_bits(B))
    dA, dB = d(Ah).half(), d(Bh).half()
    dC = torch.zeros(c["M"], c["N"], dtype=torch.float16, device=dev)
    rc = R.ref_fp16_mm_f16(_vp(dA.data_ptr()), _vp(dB.data_ptr()), _vp(dC.data_ptr()), c["M"], c["N"], c["K"], None)
    torch.cuda.synchronize()
    ref_h = dC.float().cpu().numpy()
    exact = o.exact_gemm(Ah, Bh)
    summary["ref_fp16_rc"] = int(rc)
    summary["ref_fp16_max_abs_err_vs_exact"] = float(np.abs(ref_h - exact).max())
    summary["ref_fp16_equals_rounded_exact"] = float((o.to_f16_bits(exact.astype(np.float32)) == o.to_f16_bits(ref_h)).mean())
    arrays["fp16_C_bits"] = o.to_f16_bits(ref_h)

    # 4. reference FP8 fused-quant kernels (examples/005.fp8.mm.cu)
    c = PIN_CASES["fp8"]
    M, N, K = c["M"], c["N"], c["K"]
    x, w = inputs_fp8(c["seed"], M, N, K)
    A_q, A_s = o.quant_1x128(x)
    B_q, B_s = o.quant_128x128(w)
    t1_q, t1_s, t1_acc = o.fp8_blockwise_mm(A_q, A_s, B_q, B_s)
    t0 = o.fp8_blockwise_acc(A_q, A_s, B_q, B_s, exact=True)
    dAq, dAs, dBq, dBs = d(A_q), d(A_s), d(B_q), d(B_s)
    for name in ("ref_fp8_mm_v1", "ref_fp8_mm_opt_reg", "ref_fp8_mm_inner_split"):
        dCq = torch.zeros(M, N, dtype=torch.uint8, device=dev)
        dCs = torch.zeros(N // 128, M, dtype=torch.float32, device=dev)
        rc = getattr(R, name)(_vp(dAq.data_ptr()), _vp(dAs.data_ptr()), _vp(dBq.data_ptr()), _vp(dBs.data_ptr()),
                              _vp(dCq.data_ptr()), _vp(dCs.data_ptr()), M, N, K, None)
        torch.cuda.synchronize()
        cq, cs = dCq.cpu().numpy(), dCs.cpu().numpy()
        deq = o.dequant_1x128(cq, cs)
        key = name[len("ref_"):]
        summary[key] = dict(
            rc=int(rc),
            q_equal_oracle=float((cq == t1_q).mean()),
            scale_equal_oracle=float((cs.view(np.uint32) == t1_s.view(np.uint32)).mean()),
            scale_max_rel_diff=float(np.abs(cs / t1_s - 1).max()),
            eps_ref_max_abs_vs_T0=float(np.abs(deq - t0).max()),
            eps_ref_over_amax=float(np.abs(deq - t0).max() / np.abs(t0).max()),
            oracle_deq_max_abs_vs_T0=float(np.abs(o.dequant_1x128(t1_q, t1_s) - t0).max()),
        )
        if name == "ref_fp8_mm_opt_reg":  # one variant is kept as golden vector; the others only in the summary
            arrays[key + "_Cq"], arrays[key + "_Cs"] = cq, cs
    dC = torch.zeros(M, N, dtype=torch.float32, device=dev)
    rc = R.ref_fp8_mm_f32out(_vp(dAq.data_ptr()), _vp(dAs.data_ptr()), _vp(dBq.data_ptr()), _vp(dBs.data_ptr()),
                             _vp(dC.data_ptr()), M, N, K, None)
    torch.cuda.synchronize()
    f32 = dC.cpu().numpy()
    summary["fp8_mm_f32out"] = dict(rc=int(rc), max_abs_vs_T1=float(np.abs(f32 - t1_acc).max()),
                                    max_abs_vs_T0=float(np.abs(f32 - t0).max()), amax=float(np.abs(t0).max()))
    arrays["fp8_mm_f32out_C_rows0_64"] = f32[:64]

    summary["cases"] = PIN_CASES
    summary["device"] = torch.cuda.get_device_name(0)
    np.savez_compressed(out / "ref_pins.npz", **arrays)
    (out / "ref_pins.json").write_text(json.dumps(summary, indent=1))
    print(json.dumps(summary, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
