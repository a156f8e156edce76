"""B200-native (sm_100a) long-context decode attention kernels behind the ``sparse_kv`` API.

Public surface (same names as the reference package ``sparse_kv``,
sparse_kv/__init__.py:4-16): ``sparse_attention``, ``fused_kv_evict``,
``kv_evict_quant_forward`` and ``CUDA_AVAILABLE``; the extension-module
functions live in ``_C`` (``fused_gqa``, ``sparse_attention_forward``,
``kv_evict_quant_forward``).  ``install_as_sparse_kv()`` registers this package
under the name ``sparse_kv`` so that reference call sites import it unchanged.
"""
from __future__ import annotations

import sys

from . import _lib

__version__ = "0.1.0"


def _cuda_available() -> bool:
    try:
        import torch
        return _lib.LIB_PATH.exists() and torch.cuda.is_available()
    except Exception:  # pragma: no cover - torch missing or broken
        return False


CUDA_AVAILABLE = _cuda_available()

from . import _C, attention, eviction  # noqa: E402
from ._C import fused_gqa, kv_evict_quant_forward, sparse_attention_forward  # noqa: E402
from .attention import sparse_attention  # noqa: E402
from .eviction import fused_kv_evict  # noqa: E402

__all__ = ["sparse_attention", "fused_kv_evict", "kv_evict_quant_forward", "sparse_attention_forward", "fused_gqa", "CUDA_AVAILABLE",
           "install_as_sparse_kv"]


def install_as_sparse_kv() -> None:
    """Make ``import sparse_kv`` and ``from sparse_kv._C import ...`` resolve to this package."""
    me = sys.modules[__name__]
    sys.modules["sparse_kv"] = me
    sys.modules["sparse_kv._C"] = _C
    for sub in ("attention", "eviction"):
        mod = sys.modules.get(f"{__name__}.{sub}")
        if mod is not None:
            sys.modules[f"sparse_kv.{sub}"] = mod
