"""``sparse_attention`` with the reference's signature (sparse_kv/attention.py:5-22)."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _C


def sparse_attention(Q: Tensor, K: Tensor, V: Tensor, top_k: int = 64, sink_tokens: int = 4) -> Tensor:
    """Token-sparse attention: softmax over the ``top_k`` best keys plus the first ``sink_tokens``.

    Q ``[B,H,S,D]``, K/V ``[B,H,T,D]`` of any float dtype on a CUDA device; computed in fp16 storage /
    fp32 arithmetic by the sm_100a kernels and returned in Q's dtype, as the reference's CUDA branch
    does (sparse_kv/attention.py:13-20).  Unlike that branch, ``sink_tokens`` is honoured, matching
    ``_reference_sparse_attention`` (sparse_kv/attention.py:25-38).  There is no PyTorch fallback:
    CPU tensors raise ``RuntimeError``.
    """
    orig = Q.dtype
    out = _C.token_sparse_decode(Q.to(torch.float16), K.to(torch.float16), V.to(torch.float16), top_k, sink_tokens)
    return out.to(orig)
