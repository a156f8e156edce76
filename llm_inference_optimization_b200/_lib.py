"""ctypes binding of ``csrc/libskv_b200.so`` (the C-ABI declared in ``include/skv_b200.h``).

There is no CPU fallback behind these calls: if the shared object is missing
the loader raises, and every entry point returns a non-zero status (turned into
``RuntimeError`` here) when no CUDA device can run it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# SKV_B200_LIB points the loader at another build of the same library (for example an instrumented one).
LIB_PATH = Path(os.environ.get("SKV_B200_LIB") or Path(__file__).resolve().parent / "csrc" / "libskv_b200.so")

KV_F16, KV_I8, KV_E4M3 = 0, 1, 2
QUANT_NONE, QUANT_INT8, QUANT_E4M3, QUANT_CAST = 0, 1, 2, 3
ORDER_POSITION, ORDER_SCORE = 0, 1

_vp, _i, _ll, _f, _sz = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/skv_b200.h one to one.
SIGNATURES = {
    "skv_last_error": (C.c_char_p, []),
    "skv_abi_version": (_i, []),
    "skv_workspace_status": (_i, [_vp, _i, _vp, C.POINTER(_i)]),
    "skv_gqa_set_tuning": (_i, [_i, _i]),
    "skv_gqa_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "skv_gqa_decode_splits": (_i, [_i, _i, _i, _i, _i, _i]),
    "skv_gqa_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _vp, _vp,
                            _ll, _ll, _ll, _vp, _f, _i, _vp]),
    "skv_gqa_decode_mass_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "skv_gqa_decode_mass": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _ll, _ll, _ll, _vp, _f, _i, _vp]),
    "skv_token_sparse_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "skv_token_sparse_set_mma_scores": (_i, [_i]),
    "skv_token_sparse_set_stagger": (_i, [_i]),
    "skv_token_sparse_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i,
                                     _ll, _ll, _ll, _ll, _ll, _ll, _i, _i, _f, _i, _vp]),
    "skv_block_sparse_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "skv_block_sparse_set_mma_scores": (_i, [_i]),
    "skv_block_sparse_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i,
                                     _ll, _ll, _ll, _ll, _ll, _i, _i, _f, _i, _vp]),
    "skv_kv_evict_keep_count": (_i, [_i, _i, _i]),
    "skv_kv_evict_set_fused": (_i, [_i]),
    "skv_kv_evict_quant": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll,
                                _i, _i, _i, _i, _i, _vp]),
    "skv_gqa_set_q8_stages": (_i, [_i]),
    "skv_gqa_set_ragged_worklist": (_i, [_i]),
    "skv_gqa_set_q8_two_per_sm": (_i, [_i]),
    "skv_gqa_set_early_kv": (_i, [_i]),
    "skv_gqa_set_cluster_combine": (_i, [_i]),
    "skv_gqa_decode_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i,
                                  _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _f, _i, _vp]),
    "skv_quest_num_blocks": (_i, [_i, _i]),
    "skv_quest_set_ring_scores": (_i, [_i]),
    "skv_quest_set_fused": (_i, [_i]),
    "skv_quest_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "skv_quest_build_meta": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                                  _ll, _ll, _ll, _ll, _ll, _vp, _i, _vp]),
    "skv_quest_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i,
                              _i, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _f, _i, _vp]),
    "skv_residual_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _vp]),
    "skv_allreduce_residual_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _i, C.c_uint, _i, _vp]),
    "skv_allreduce_residual_rmsnorm_push": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _i, C.c_uint, _i, _vp]),
    "skv_skinny_gemm_set_min_blocks": (_i, [_i]),
    "skv_skinny_gemm_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "skv_skinny_gemm": (_i, [_vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _vp]),
    "skv_silu_mul": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "skv_rope_quant_append": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i,
                                   _ll, _ll, _ll, _ll, _ll, _f, _vp, _i, _i, _i, _vp, _i, _vp]),
    "skv_gqa_decode_noalloc_status": (_i, [_i, _vp, C.POINTER(_i)]),
    "skv_gqa_decode_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll, _ll, _ll, _vp, _f, _i, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared object once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m llm_inference_optimization_b200.build` "
                "(needs nvcc). There is no CPU fallback.")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().skv_last_error().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    """Turn a non-zero C-ABI status into the RuntimeError the reference raises via TORCH_CHECK."""
    if status != 0:
        raise RuntimeError(f"{what} failed (status {status}): {last_error()}")
