"""Builds the C-ABI shared library `libinpc_b200.so` in-tree with nvcc for sm_100a.

    python -m inpc_b200._build [--force]
    python -m inpc_b200._build --checked    # libinpc_b200_checked.so: every gather index range-checked (debugging aid)

The library has no dependency on torch or Python; the Python package binds it with ctypes.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libinpc_b200.so"
LIB_CHECKED = PKG / "libinpc_b200_checked.so"    # select it with INPC_B200_LIB=<path>
OBJ = PKG / "csrc" / "_obj"
SOURCES = ["api.cu", "radix_sort.cu", "raster.cu", "sampler.cu", "misc.cu", "octree.cu"]
HEADERS = [CSRC / "common.cuh", PKG.parent / "include" / "inpc_b200.h"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def needs_build(lib: Path = LIB) -> bool:
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [CSRC / s for s in SOURCES] + HEADERS)


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    """Compiles the library; `checked` builds the variant whose kernels range-check every index they
    gather with and report violations through a status word (about 2 % slower)."""
    lib = LIB_CHECKED if checked else LIB
    if not force and not needs_build(lib):
        return lib
    obj_dir = OBJ / "checked" if checked else OBJ
    obj_dir.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    extra = ["-DINPC_CHECK_INDICES"] if checked else []

    def compile_one(src: str) -> Path:
        obj = obj_dir / (src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    tmp = lib.with_suffix(".so.tmp")
    subprocess.check_call([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp),
                           *map(str, objs)])
    os.replace(tmp, lib)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv))
