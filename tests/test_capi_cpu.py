"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
header declares, validates arguments before touching a device, and refuses to
compute without an sm_100 GPU (there is no CPU path to fall back to)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "llmmm_c.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llmmm_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(capi):
    L = capi.lib()
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/llmmm_c.h but not exported"
    assert set(capi.EXPORTED_SYMBOLS) <= set(names)


def test_version_and_error_text(capi):
    L = capi.lib()
    assert b"sm_100a" in L.llmmm_version()
    assert isinstance(L.llmmm_last_error(), bytes)


def test_shape_validation_needs_no_device(capi):
    L = capi.lib()
    one = ctypes.c_void_p(0x1000)
    # reference launchers throw "M or N or K are not aligned." (src/mm/fp16/mm.cu:19-21)
    assert L.llmmm_fp16_mm_f16(one, one, one, 256, 255, 256, None) == 1
    assert b"not aligned" in L.llmmm_last_error()
    assert L.llmmm_fp16_mm_bf16(one, one, one, 0, 256, 256, None) == 1
    assert L.llmmm_fp16_mm_f16(None, one, one, 256, 256, 256, None) == 1
    assert L.llmmm_fp16_mm_f16(ctypes.c_void_p(0x1001), one, one, 256, 256, 256, None) == 1
    assert L.llmmm_fp8_blockwise_mm_e4m3out(one, one, one, one, one, one, 128, 100, 128, None) == 1
    assert L.llmmm_fp8_blockwise_mm_e4m3out(one, one, one, one, one, one, 128, 128, 200, None) == 1
    assert L.llmmm_fp8_blockwise_mm_f32out(one, one, one, one, one, 0, 128, 128, None) == 1
    assert L.llmmm_fp8_quant_1x128(one, one, one, 4, 100, None) == 1
    assert L.llmmm_fp8_quant_128x128(one, one, one, 100, 128, None) == 1


def test_workspace_size_rule(capi):
    # decode-sized problems need scratch; larger M does not
    assert capi.fp8_workspace_bytes(1, 6144, 2560) == capi.fp8_workspace_bytes(16, 2560, 9728) > 0
    assert capi.fp8_workspace_bytes(64, 6144, 2560) > capi.fp8_workspace_bytes(32, 6144, 2560)
    # more than 64 rows: one size for all shapes (partial tiles of the pair kernel's split last wave)
    assert capi.fp8_workspace_bytes(4096, 4096, 4096) == capi.fp8_workspace_bytes(65, 128, 128) > 0
    assert capi.fp8_workspace_bytes(128, 6144, 2560) == capi.fp8_workspace_bytes(129, 128, 128)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour on a machine without a GPU")
def test_compute_fails_loudly_without_gpu(capi):
    L = capi.lib()
    one = ctypes.c_void_p(0x1000)
    assert L.llmmm_fp16_mm_f16(one, one, one, 256, 256, 256, None) == 2
    assert L.llmmm_last_error() != b""
    assert L.llmmm_fp8_blockwise_mm_e4m3out(one, one, one, one, one, one, 128, 128, 128, None) == 2
    assert L.llmmm_fp8_quant_1x128(one, one, one, 4, 128, None) == 2
    with pytest.raises(RuntimeError):
        capi.fp16_mm(torch.zeros(1), torch.zeros(1), torch.zeros(1), 1, 8, 8)


def test_python_wrapper_rejects_unsupported_dtype(capi):
    with pytest.raises(RuntimeError, match="T is not supported"):
        capi.fp16_mm(torch.zeros(8, 8), torch.zeros(8, 8), torch.zeros(8, 8), 8, 8, 8)


def test_build_refuses_spilling_gemm_kernels():
    # a few spilled bytes in the FP8 promotion loop cost a third of the speed: the build parses ptxas -v
    from llmmm_b200.build import spilling_kernels
    log = "\n".join([
        "ptxas info    : Compiling entry function '_ZN5llmmm30fp8_blockwise_gemm_pair_kernelILb0EEEv' for 'sm_100a'",
        "ptxas info    : Function properties for _ZN5llmmm30fp8_blockwise_gemm_pair_kernelILb0EEEv",
        "    16 bytes stack frame, 12 bytes spill stores, 52 bytes spill loads",
        "ptxas info    : Compiling entry function '_ZN5llmmm25fp8_blockwise_gemm_kernelILb1EEEv' for 'sm_100a'",
        "ptxas info    : Function properties for _ZN5llmmm25fp8_blockwise_gemm_kernelILb1EEEv",
        "    8 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads",
        "ptxas info    : Compiling entry function '_ZN5llmmm18quant_1x128_kernelEPKfPhPfii' for 'sm_100a'",
        "ptxas info    : Function properties for _ZN5llmmm18quant_1x128_kernelEPKfPhPfii",
        "    16 bytes stack frame, 12 bytes spill stores, 52 bytes spill loads",
    ])
    assert spilling_kernels(log, ("fp8_blockwise_gemm",)) == ["_ZN5llmmm30fp8_blockwise_gemm_pair_kernelILb0EEEv"]


def test_describe_plan_and_tune_validate_before_touching_a_device(capi):
    L = capi.lib()
    buf = ctypes.create_string_buffer(256)
    n = ctypes.c_size_t(len(buf))
    assert L.llmmm_describe_plan(7, 256, 256, 256, buf, n) == 2 and b"not supported" in L.llmmm_last_error()
    assert L.llmmm_describe_plan(capi.KINDS["fp8"], 256, 100, 256, buf, n) == 1 and b"not aligned" in L.llmmm_last_error()
    assert L.llmmm_describe_plan(capi.KINDS["fp16"], 256, 256, 12, buf, n) == 1
    assert L.llmmm_describe_plan(capi.KINDS["fp16"], 256, 256, 256, None, n) == 1
    # valid arguments, but this machine has no sm_100 device: unsupported, never a made-up answer
    assert L.llmmm_describe_plan(capi.KINDS["fp8"], 4096, 4096, 4096, buf, n) == 2 and buf.value == b""
    assert L.llmmm_tune(capi.KINDS["bf16"], 4096, 4096) == 2
    assert L.llmmm_tune(9, 4096, 4096) == 2
