"""Runs one shape on the profiling build of the library and prints the in-kernel time stamps.

    python -m llmmm_b200.build --profile
    python -m llmmm_b200.profile_dump fp8 M N K        # FP8 blockwise GEMM, e4m3 output (decode kernel for M <= 64)
    python -m llmmm_b200.profile_dump fp16 M N K
    python -m llmmm_b200.profile_dump rope M N K       # qkv projection with the q/k-norm + RoPE epilogue; heads of
                                                       # 128 columns split 4 : 1 : 1 into query, key and value heads

The profiling build (libllmmm_b200_profile.so, -DLLMMM_PROFILE) records %globaltimer / clock64 values at the
hand-off points of its kernels and exports llmmm_profile_dump_* functions that print them; the regular library
contains none of this.  The figures quoted under profiles/ as "in-kernel stamps" come from this module.  The
stamps cost time themselves (tens of nanoseconds each): use them for the order and rough size of the phases,
not for absolute kernel times.
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import torch

LIB = Path(__file__).resolve().parent / "libllmmm_b200_profile.so"


def main(argv: list[str]) -> int:
    if len(argv) != 4 or argv[0] not in ("fp8", "fp16", "rope"):
        print(__doc__)
        return 2
    if not LIB.exists():
        print(f"{LIB} is missing: build it with `python -m llmmm_b200.build --profile`")
        return 1
    kind, (M, N, K) = argv[0], map(int, argv[1:])
    L = ctypes.CDLL(str(LIB))
    vp = ctypes.c_void_p
    dev = torch.device("cuda", 0)
    stream = vp(torch.cuda.current_stream().cuda_stream)
    L.llmmm_fp8_workspace_bytes.restype = ctypes.c_size_t
    L.llmmm_last_error.restype = ctypes.c_char_p
    need = max(L.llmmm_fp8_workspace_bytes(M, N, K), L.llmmm_fp8_workspace_bytes(4096, 4096, 4096))
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    L.llmmm_set_workspace(vp(ws.data_ptr()), ctypes.c_size_t(need))
    if kind == "fp16":
        A = torch.randn(M, K, device=dev).half()
        B = torch.randn(K, N, device=dev).half()
        C = torch.empty(M, N, device=dev, dtype=torch.float16)
        call = lambda: L.llmmm_fp16_mm_f16(vp(A.data_ptr()), vp(B.data_ptr()), vp(C.data_ptr()), M, N, K, stream)
        dumps = ("llmmm_profile_dump16",)
    else:
        A = torch.randint(0, 120, (M, K), dtype=torch.uint8, device=dev)
        As = torch.rand(K // 128, M, device=dev)
        B = torch.randint(0, 120, (N, K), dtype=torch.uint8, device=dev)
        Bs = torch.rand(N // 128, K // 128, device=dev)
        C = torch.empty(M, N, dtype=torch.uint8, device=dev)
        Cs = torch.empty(N // 128, M, device=dev)
        L.llmmm_set_static_weights(1)
        if kind == "rope":
            heads = N // 128
            if N % 768 != 0:
                print("rope: N must be a multiple of 768 (4 : 1 : 1 heads of 128 columns)")
                return 2
            n_kv, n_q = heads // 6, 4 * (heads // 6)
            ang = torch.arange(8192, device=dev, dtype=torch.float32)[:, None] / (1e6 ** (torch.arange(64, device=dev) / 64.0))[None, :]
            cos_t, sin_t = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
            pos = ((torch.arange(M, device=dev, dtype=torch.int32) * 7 + 17) % 8192).contiguous()
            qw, kw = torch.rand(128, device=dev) + 0.5, torch.rand(128, device=dev) + 0.5
        rope_call = lambda: L.llmmm_fp8_blockwise_mm_qk_norm_rope_e4m3out(
            vp(A.data_ptr()), vp(As.data_ptr()), vp(B.data_ptr()), vp(Bs.data_ptr()), vp(C.data_ptr()), vp(Cs.data_ptr()),
            vp(pos.data_ptr()), vp(cos_t.data_ptr()), vp(sin_t.data_ptr()), 8192, vp(qw.data_ptr()), vp(kw.data_ptr()),
            ctypes.c_float(1e-6), n_q, n_kv, M, N, K, stream)
        call = rope_call if kind == "rope" else lambda: L.llmmm_fp8_blockwise_mm_e4m3out(vp(A.data_ptr()), vp(As.data_ptr()), vp(B.data_ptr()), vp(Bs.data_ptr()),
                                                        vp(C.data_ptr()), vp(Cs.data_ptr()), M, N, K, stream)
        dumps = ("llmmm_profile_dump_decode",) if M <= 64 else ("llmmm_profile_dump8", "llmmm_profile_stamps8")
    for _ in range(8):  # a chain of launches: the stamps are those of the last one
        if call() != 0:
            print(L.llmmm_last_error().decode())
            return 1
    torch.cuda.synchronize()
    for name in dumps:
        getattr(L, name)()
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
