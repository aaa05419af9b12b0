"""Builds libllmmm_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python -m llmmm_b200.build [--force] [--verbose] [--profile]

--profile builds a second library, libllmmm_b200_profile.so, from the same sources with -DLLMMM_PROFILE: the
kernels then record %globaltimer / clock64 stamps at their hand-off points and the library exports
llmmm_profile_dump_* functions that print them (load that library instead of the regular one, run the shape,
call the dump function).  The regular library contains none of this.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libllmmm_b200.so"
PROFILE_LIB = PKG / "libllmmm_b200_profile.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


# Kernels whose hot loop has no register to spare: the build fails if ptxas reports spills for them.
NO_SPILL = ("fp8_blockwise_gemm",)
# (no instantiation is exempt)
SPILL_TOLERATED: tuple[str, ...] = ()


def spilling_kernels(ptxas_log: str, patterns: tuple[str, ...]) -> list[str]:
    """Entry functions matching `patterns` for which `-Xptxas -v` reports spill stores or loads."""
    bad, current = [], None
    for line in ptxas_log.splitlines():
        if "Compiling entry function" in line or "Function properties for" in line:
            current = line.split("'")[1] if "'" in line else line.rsplit(" ", 1)[-1]
        elif "bytes spill stores" in line and current and any(p in current for p in patterns):
            if "0 bytes spill stores, 0 bytes spill loads" not in line and not any(t in current for t in SPILL_TOLERATED):
                bad.append(current)
    return sorted(set(bad))


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


def build_library(force: bool = False, verbose: bool = False, profile: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "llmmm_c.h"]
    obj_dir = OBJ / "profile" if profile else OBJ
    lib = PROFILE_LIB if profile else LIB
    flags = FLAGS + (["-DLLMMM_PROFILE"] if profile else [])
    obj_dir.mkdir(parents=True, exist_ok=True)

    def compile_one(src: Path) -> tuple[Path, str]:
        obj = obj_dir / (src.stem + ".o")
        if not force and _newer(obj, [src] + headers):
            return obj, ""
        cmd = [NVCC, *flags, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        spilled = [] if profile else spilling_kernels(r.stderr, NO_SPILL)
        if spilled:
            obj.unlink(missing_ok=True)
            raise RuntimeError(f"{src.name}: ptxas spilled registers in {spilled}; these kernels lose a third of their "
                               "speed to a few spilled bytes (change the setmaxnreg split until -Xptxas -v shows 0)")
        return obj, r.stderr

    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    if force or not _newer(lib, objs):
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv, profile="--profile" in sys.argv))
