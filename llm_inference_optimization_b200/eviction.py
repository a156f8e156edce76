"""``fused_kv_evict`` with the reference's signature (sparse_kv/eviction.py:12-27)."""
from __future__ import annotations

from typing import NamedTuple

import torch
from torch import Tensor

from . import _C, _lib

_QUANT = {None: _lib.QUANT_NONE, "none": _lib.QUANT_NONE, "int8": _lib.QUANT_INT8, "fp8": _lib.QUANT_E4M3,
          "e4m3": _lib.QUANT_E4M3, "cast": _lib.QUANT_CAST}
_ORDER = {"position": _lib.ORDER_POSITION, "score": _lib.ORDER_SCORE}


class EvictionResult(NamedTuple):
    K: Tensor                 # [B,H,keep,D] codes (int8 / float8_e4m3fn) or rows in the cache dtype
    V: Tensor
    k_scale: Tensor | None    # [B,H,keep] fp32 for the scaled modes
    v_scale: Tensor | None
    indices: Tensor           # [B,H,keep] int32 positions of the kept tokens


def fused_kv_evict(K_cache: Tensor, V_cache: Tensor, attn_scores: Tensor, top_k: int, use_int8: bool = True, *,
                   recent_tokens: int = 0, quant: str | None = None, order: str | None = None,
                   return_aux: bool = False):
    """Keep the ``top_k`` highest-scoring tokens of a KV cache, compact them and optionally quantise.

    ``K_cache``/``V_cache`` ``[B,H,T,D]``, ``attn_scores`` ``[B,H,T]``.  Called exactly like the reference
    (no keyword arguments) it returns what ``_reference_eviction`` returns (sparse_kv/eviction.py:30-44):
    rows in descending-score order, cast to int8 by truncation when ``use_int8``.  Keyword-only extensions:

    * ``recent_tokens``: the last n positions are kept in addition to the ``top_k`` best of the rest;
    * ``quant``: ``"int8"`` (symmetric, scale = amax/127) or ``"fp8"`` (E4M3, scale = amax/448) with one fp32
      scale per token and head; ``"cast"`` is the reference's unscaled cast; ``"none"`` copies rows;
    * ``order``: ``"position"`` (cache order, the compacted-cache layout) or ``"score"`` (topk order);
      defaults to ``"score"`` unless ``quant`` is a scaled mode or ``recent_tokens`` is given;
    * ``return_aux``: return an ``EvictionResult`` with scales and kept positions instead of ``(K, V)``.
    """
    _C._require(K_cache.is_cuda and V_cache.is_cuda and attn_scores.is_cuda, "K/V/scores must be CUDA tensors")
    _C._require(K_cache.dim() == 4 and V_cache.shape == K_cache.shape, "K_cache and V_cache must both be [B,H,T,D]")
    B, H, T, D = K_cache.shape
    _C._require(attn_scores.shape == (B, H, T), "attn_scores must be [B,H,T]")
    _C._require(top_k >= 0 and recent_tokens >= 0, "top_k and recent_tokens must not be negative")
    if quant is None:
        quant = "cast" if use_int8 else "none"
    _C._require(quant in _QUANT, f"unknown quant mode {quant!r}")
    mode = _QUANT[quant]
    if order is None:
        order = "position" if (mode in (_lib.QUANT_INT8, _lib.QUANT_E4M3) or recent_tokens > 0) else "score"
    _C._require(order in _ORDER, f"unknown order {order!r}")
    orig = K_cache.dtype
    K16, V16 = K_cache.to(torch.float16), V_cache.to(torch.float16)
    sc = attn_scores.to(torch.float32).contiguous()
    sb, sh, st = _C._kv_strides(K16, V16, "fused_kv_evict")
    lib = _lib.load()
    dev = _C._dev_index(K16)
    keep = lib.skv_kv_evict_keep_count(T, int(top_k), int(recent_tokens))
    _C._require(keep > 0, "nothing to keep")
    idx = torch.empty((B, H, keep), dtype=torch.int32, device=K16.device)
    if mode == _lib.QUANT_NONE:
        Ko = torch.empty((B, H, keep, D), dtype=torch.float16, device=K16.device)
        Vo = torch.empty_like(Ko)
    else:
        Ko = torch.empty((B, H, keep, D), dtype=torch.int8, device=K16.device)
        Vo = torch.empty_like(Ko)
    ks = vs = None
    if mode in (_lib.QUANT_INT8, _lib.QUANT_E4M3):
        ks = torch.empty((B, H, keep), dtype=torch.float32, device=K16.device)
        vs = torch.empty_like(ks)
    stream = torch.cuda.current_stream(K16.device).cuda_stream
    rc = lib.skv_kv_evict_quant(K16.data_ptr(), V16.data_ptr(), sc.data_ptr(), idx.data_ptr(), Ko.data_ptr(),
                                Vo.data_ptr(), None if ks is None else ks.data_ptr(),
                                None if vs is None else vs.data_ptr(), B, H, T, D, sb, sh, st, int(top_k),
                                int(recent_tokens), mode, _ORDER[order], dev, stream)
    _lib.check(rc, "fused_kv_evict")
    if mode == _lib.QUANT_NONE:
        Ko, Vo = Ko.to(orig), Vo.to(orig)
    elif mode == _lib.QUANT_E4M3:
        Ko, Vo = Ko.view(torch.float8_e4m3fn), Vo.view(torch.float8_e4m3fn)
    if return_aux:
        return EvictionResult(Ko, Vo, ks, vs, idx)
    return Ko, Vo


class AttentionMassPolicy:
    """Eviction policy loop: accumulate every token's attention mass while decoding, evict on demand.

    ``decode(Q, K, V, scale)`` is ``fused_gqa`` with the mass output switched on: each call adds, per cached
    token, the attention probability summed over the query heads of its kv-head into ``self.mass``
    (``[B, Hkv, N]`` fp32).  ``evict(K, V, budget, ...)`` hands that running score to ``fused_kv_evict`` -- the
    argument the reference leaves to its caller to produce (sparse_kv/eviction.py:12-22) -- and clears it.
    K and V use the decode layout ``[B, N, Hkv, D]``; the eviction call sees them as ``[B, Hkv, N, D]`` views.
    """

    def __init__(self, batch: int, kv_heads: int, max_tokens: int, device):
        self.mass = torch.zeros((batch, kv_heads, max_tokens), dtype=torch.float32, device=device)
        self.steps = 0

    def decode(self, Q: Tensor, K: Tensor, V: Tensor, scale: float, *, seq_lens: Tensor | None = None) -> Tensor:
        _C._require(K.shape[1] == self.mass.shape[2], "the cache length must equal the accumulator's max_tokens")
        out = _C.fused_gqa(Q, K, V, scale, seq_lens=seq_lens, mass=self.mass)
        self.steps += 1
        return out

    def evict(self, K: Tensor, V: Tensor, budget: int, *, recent_tokens: int = 0, quant: str = "int8", **kw):
        """``fused_kv_evict`` on the accumulated mass; returns its result and resets the accumulator."""
        res = fused_kv_evict(K.permute(0, 2, 1, 3), V.permute(0, 2, 1, 3), self.mass, budget,
                             recent_tokens=recent_tokens, quant=quant, **kw)
        self.mass.zero_()
        self.steps = 0
        return res
