"""Recipe: compile the REFERENCE project's own CUDA kernels, unchanged, for sm_100a.

TEST INFRASTRUCTURE, not product code.  The three kernel files and the pybind file of the
reference (csrc/kernels/{gqa_decode,sparse_attention,kv_evict_quant}.cu, csrc/pybind/bindings.cpp)
are compiled from where they lie in the reference checkout -- no source is copied -- with the
flags of the reference's setup.py:10-19 except for the architecture (`-arch=sm_90a` there,
sm_100a here; the sources use nothing Hopper-specific).  The result is a torch extension module
`sparse_kv_ref_C` under `oracle/_ref/` (git-ignored), exposing the reference's three functions
(csrc/pybind/bindings.cpp:26-31): `fused_gqa`, `sparse_attention_forward`, `kv_evict_quant_forward`.

It serves two purposes, both outside the product path:
  * `tests/golden/make_refcuda_golden.py` runs it on a B200 and records outputs that pin the
    oracle's block-mean rule and dense decode to the reference's own kernels;
  * the benchmark harness times it beside this library's kernels on the same GPU.

    python oracle/build_ref.py [/path/to/reference/checkout]

`load()` imports an already built module and never compiles: the machine that runs the GPU
tests has the built file but not the reference checkout.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
MODULE = "sparse_kv_ref_C"
# the reference checkout: SKV_REFERENCE_DIR, else a directory `reference` beside this repository
DEFAULT_REFERENCE = Path(os.environ.get("SKV_REFERENCE_DIR") or HERE.parent.parent / "reference")

SOURCES = [
    "csrc/pybind/bindings.cpp",
    "csrc/kernels/kv_evict_quant.cu",
    "csrc/kernels/sparse_attention.cu",
    "csrc/kernels/gqa_decode.cu",
]
# setup.py:10-19 of the reference with the architecture replaced.
NVCC_FLAGS = [
    "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math", "-lineinfo", "-DUSE_HOPPER=1",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
]
CXX_FLAGS = ["-O3", "-std=c++17"]


def built_path() -> Path | None:
    hits = sorted(OUT_DIR.glob(f"{MODULE}*.so"))
    return hits[0] if hits else None


def build(reference: Path = DEFAULT_REFERENCE, verbose: bool = False) -> Path:
    """Compile the reference's sources into oracle/_ref/; returns the module's path."""
    from torch.utils import cpp_extension

    srcs = [reference / s for s in SOURCES]
    missing = [str(s) for s in srcs if not s.exists()]
    if missing:
        raise FileNotFoundError("reference sources not found: " + ", ".join(missing))
    OUT_DIR.mkdir(exist_ok=True)
    cpp_extension.load(
        name=MODULE, sources=[str(s) for s in srcs],
        extra_include_paths=[str(reference / "csrc/kernels"), str(reference / "csrc/pybind")],
        extra_cflags=CXX_FLAGS, extra_cuda_cflags=NVCC_FLAGS, extra_ldflags=["-lcuda"],
        build_directory=str(OUT_DIR), verbose=verbose, is_python_module=False)
    path = built_path()
    if path is None:
        raise RuntimeError("the extension build produced no module under " + str(OUT_DIR))
    return path


def available() -> bool:
    return built_path() is not None


def load():
    """Import the prebuilt reference extension (torch must be imported first: it links libtorch)."""
    import torch  # noqa: F401  (loads libtorch / libc10 the module depends on)

    path = built_path()
    if path is None:
        raise RuntimeError(f"{OUT_DIR}/{MODULE}*.so is missing: run `python oracle/build_ref.py` where the "
                           "reference checkout is available")
    if MODULE in sys.modules:
        return sys.modules[MODULE]
    spec = importlib.util.spec_from_file_location(MODULE, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[MODULE] = mod
    return mod


if __name__ == "__main__":
    ref = Path(sys.argv[1]) if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else DEFAULT_REFERENCE
    print(build(ref, verbose="-v" in sys.argv))
