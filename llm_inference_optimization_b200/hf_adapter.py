"""Hugging Face Llama adapter: route the decode step of ``LlamaAttention`` through the sm_100a kernels.

The counterpart of the reference's ``patch_attention`` / ``restore_attention``
(benchmarks/llama_integration_benchmark.py:114-230, :233-245), written for transformers 5.x, where attention
back-ends are functions in a registry instead of methods to monkeypatch: ``patch_attention`` registers one
back-end and points the model's config at it.  Behaviour follows the reference:

* prefill (more than one query position) is always dense and causal, through the stock SDPA back-end;
* a decode step (one query position) of a patched layer runs ``token-sparse`` (``kv_evict_quant_forward`` over
  ``repeat_kv``-expanded heads, only when the cache holds at least ``top_k`` tokens), ``block-sparse``
  (``sparse_attention_forward``) or ``dense``; ``dense`` calls ``fused_gqa`` on the un-expanded cache (the
  reference validates that kernel separately, ``compare_gqa_vs_sdpa`` ``:394-506``) instead of SDPA;
* layers outside ``sparse_layers`` stay on SDPA; the attention mask of a decode step is ignored, as it is there.
"""
from __future__ import annotations

from typing import Iterable

import torch

BACKEND = "skv_b200"
MODES = ("token-sparse", "block-sparse", "dense")


def _repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, Hkv, T, D] -> [B, Hkv * n_rep, T, D]`` with query head ``h`` reading kv head ``h // n_rep``."""
    if n_rep == 1:
        return x
    B, Hkv, T, D = x.shape
    return x[:, :, None].expand(B, Hkv, n_rep, T, D).reshape(B, Hkv * n_rep, T, D)


def _make_backend(mode: str, top_k: int, block_size: int, top_k_blocks: int, layers: frozenset | None):
    from transformers.integrations.sdpa_attention import sdpa_attention_forward

    from . import _C

    def skv_attention(module, query, key, value, attention_mask, dropout: float = 0.0, scaling=None, **kwargs):
        B, H, S, D = query.shape
        layer = getattr(module, "layer_idx", None)
        if S != 1 or (layers is not None and layer not in layers):
            return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                          scaling=scaling, **kwargs)
        if not query.is_cuda:
            raise RuntimeError("the skv_b200 attention back-end decodes on CUDA tensors only")
        scale = float(scaling) if scaling is not None else D ** -0.5
        Hkv, T = key.shape[1], key.shape[2]
        q16 = query[:, :, 0].to(torch.float16).contiguous()                     # [B, H, D]
        if mode == "token-sparse" and T >= top_k:
            # the reference's kernel fixes the softmax scale at 1/sqrt(D) (kv_evict_quant.cu:122)
            k = _repeat_kv(key, H // Hkv).to(torch.float16).contiguous()
            v = _repeat_kv(value, H // Hkv).to(torch.float16).contiguous()
            out = _C.kv_evict_quant_forward(q16[:, :, None], k, v, top_k, False)[:, :, 0]
        elif mode == "block-sparse":
            k = _repeat_kv(key, H // Hkv).to(torch.float16).contiguous()
            v = _repeat_kv(value, H // Hkv).to(torch.float16).contiguous()
            out = _C.sparse_attention_forward(q16[:, :, None], k, v, block_size, top_k_blocks)[:, :, 0]
        else:
            # [B, Hkv, T, D] cache read in place as [B, T, Hkv, D]: the kernel takes strides, no copy
            out = _C.fused_gqa(q16, key.to(torch.float16).transpose(1, 2), value.to(torch.float16).transpose(1, 2), scale)
        return out.to(query.dtype)[:, None], None                              # [B, 1, H, D]

    return skv_attention


def patch_attention(model, mode: str = "token-sparse", top_k: int = 32, block_size: int = 64, top_k_blocks: int = 8,
                    sparse_layers: Iterable[int] | None = None) -> int:
    """Send the decode steps of ``model``'s attention layers to the kernels; returns the number of layers affected.

    Arguments as in the reference (``mode`` one of ``token-sparse``, ``block-sparse``, ``dense``;
    ``sparse_layers`` limits the patch to those layer indices).  Undo with :func:`restore_attention`.
    """
    if mode not in MODES:
        raise ValueError(f"mode must be one of {MODES}, got {mode!r}")
    if top_k <= 0 or block_size <= 0 or top_k_blocks <= 0:
        raise ValueError("top_k, block_size and top_k_blocks must be positive")
    from transformers import AttentionInterface

    n_layers = len(model.model.layers)
    layers = None if sparse_layers is None else frozenset(int(i) for i in sparse_layers)
    if layers is not None and any(i < 0 or i >= n_layers for i in layers):
        raise ValueError(f"sparse_layers must lie in [0, {n_layers})")
    AttentionInterface.register(BACKEND, _make_backend(mode, top_k, block_size, top_k_blocks, layers))
    cfg = model.config
    if getattr(cfg, "_attn_implementation", None) != BACKEND:
        model._skv_prev_attn = cfg._attn_implementation
    cfg._attn_implementation = BACKEND
    return n_layers if layers is None else len(layers)


def restore_attention(model) -> int:
    """Put back the attention back-end the model had before :func:`patch_attention`; returns the layer count."""
    prev = getattr(model, "_skv_prev_attn", None)
    if prev is None:
        return 0
    model.config._attn_implementation = prev
    del model._skv_prev_attn
    return len(model.model.layers)
