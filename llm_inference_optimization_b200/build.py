"""Builds the CUDA kernels and their C-ABI into one shared object, in-tree.

The library is plain ``nvcc -shared`` output for sm_100a: it links against the
CUDA runtime only (no libtorch, no pybind11) and is loaded with ``ctypes``.
Run ``python -m llm_inference_optimization_b200.build`` after changing a
source under ``csrc/``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB_NAME = "libskv_b200.so"
LIB_PATH = CSRC / LIB_NAME
# The same sources with -DSKV_BOUNDS: every data-dependent index is range-checked and the first violation recorded
# (a self-checking debug build; point SKV_B200_LIB at it to run any program against it).
BOUNDS_LIB_PATH = CSRC / "libskv_b200_bounds.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "--threads", "0",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build(path: Path = LIB_PATH) -> bool:
    if not path.exists():
        return True
    built = path.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` into ``csrc/libskv_b200.so`` (``bounds``: the range-checking debug library
    ``csrc/libskv_b200_bounds.so``); returns its path."""
    LIB_PATH = BOUNDS_LIB_PATH if bounds else globals()["LIB_PATH"]
    if not force and not needs_build(LIB_PATH):
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the sm_100a kernels cannot be built")
    cmd = [nvcc, *NVCC_FLAGS]
    if bounds:
        cmd += ["-DSKV_BOUNDS"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd += ["-o", str(tmp), *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, bounds="--bounds" in sys.argv)
    print(path)
