"""Runs the C++ harness drivers (tests/cpp, built by __graft_entry__.build) that
use the drop-in headers llmmm_b200/src/mm/{fp16,fp8}/mm.h with the reference's
launcher names, as a reference user's test executables would."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

BIN = Path(__file__).resolve().parent / "cpp" / "bin"


def run(exe, *args):
    path = BIN / exe
    if not path.exists():
        subprocess.run(["make", "-C", str(BIN.parent)], check=True, capture_output=True)
    r = subprocess.run([str(path), *map(str, args)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout
    return r.stdout


@pytest.mark.parametrize("shape", [(256, 256, 256), (4096, 4096, 4096)])
def test_fp16_mm_test_driver(cuda, shape):
    out = run("fp16_mm_test", *shape)
    assert "TFLOPS" in out


@pytest.mark.parametrize("shape", [(256, 512, 512), (4096, 4096, 4096), (16, 2560, 4096)])
def test_fp8_mm_test_driver(cuda, shape):
    out = run("fp8_mm_test", *shape)
    assert "TFLOPS" in out


def test_transpose_test_driver(cuda):
    """The reference's transpose test (test/transpose_matrix__aligned_128_test.cc), same shapes and the same
    element-by-element memcmp, against the drop-in header llmmm_b200/src/base/base.h."""
    out = run("transpose_matrix__aligned_128_test")
    assert out.count("error =     0") == 6
