"""Build ``libdimq_b200.so`` in-tree with plain ``nvcc`` for sm_100a.

The library is header-light (no torch, no pybind): each ``csrc/*.cu`` compiles in
seconds, and the resulting shared object sits next to this file so that it
travels with the source tree.
"""

from __future__ import annotations

import os
import shutil
import sys
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libdimq_b200.so"
SOURCES = ["pack.cu", "lut_generic.cu", "lut_stream.cu", "lut_mma_stream.cu", "lut_mma_regs.cu", "lut_gemm_tc.cu", "lut_expand_gemm.cu", "aux.cu", "conv_static.cu", "a4_tc.cu", "c_api.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; dimq_b200 needs the CUDA toolkit to build its sm_100a kernels")


def _stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + [PKG.parent / "include" / "dimq_b200.h"])
    return newest > LIB.stat().st_mtime


def build(force: bool = False, verbose: bool = False, diag: bool = False) -> Path:
    """Compile every kernel source and link the shared library (no-op when up to date).

    ``diag=True`` builds ``libdimq_b200_diag.so`` instead: the same library with
    ``-DDIMQ_B200_DIAG`` (per-role cycle counters and role-skipping switches of the
    tcgen05 kernel, set through ``dimq_diag_configure``).  Nothing in the package
    loads that file; it is for kernel development.
    """
    if diag:
        return _build(PKG / "libdimq_b200_diag.so", PKG / "build_diag", ["-DDIMQ_B200_DIAG"], verbose)
    if not force and not _stale():
        return LIB
    return _build(LIB, PKG / "build", [], verbose)


def _build(lib: Path, objdir: Path, extra: list[str], verbose: bool) -> Path:
    nvcc = _nvcc()
    objdir.mkdir(exist_ok=True)

    def compile_one(src: str) -> Path:
        obj = objdir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", str(lib), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib


if __name__ == "__main__":
    print(build(force=True, verbose=bool(os.environ.get("DIMQ_BUILD_VERBOSE")), diag="--diag" in sys.argv))
