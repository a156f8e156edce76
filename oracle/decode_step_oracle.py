"""fp32 CPU restatement of one Llama-architecture decode step.  TEST INFRASTRUCTURE ONLY.

Follows the step the reference times on its Hugging Face model (benchmarks/llama_integration_benchmark.py:266-279
with the attention of :152-213): RMSNorm, q/k/v projections, rotate-half RoPE, attention of the new token over the
cached keys/values plus itself, o_proj, SwiGLU MLP, final norm and lm_head.  The KV history is passed dequantised
and unpaged; the new token's k/v go through the same FP8-E4M3 row quantisation the cache applies (no reference
counterpart for that part), so that the only differences from the product path are GEMM precision and paging.
"""
from __future__ import annotations

import math

import torch

from . import skv_oracle


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope(x, pos, theta):
    """Rotate-half rotary embedding of ``x [B, H, D]`` (fp32) at integer positions ``pos [B]``: channel d pairs with
    d + D/2, angle ``pos * theta^(-2d/D)`` -- the form of the Hugging Face Llama model the reference patches
    (benchmarks/llama_integration_benchmark.py:152-160)."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
    rot = torch.cat([-x[..., D // 2:], x[..., :D // 2]], -1)
    return x * cos + rot * sin


def quest_attention(q, K, V, lens, block: int, top_k: int, scale: float):
    """Block-sparse attention of one layer, sequence by sequence (no reference counterpart; the rule is the one of
    ``skv_oracle.quest_block_scores``): min/max metadata of the sequence's own tokens, upper-bound block scores per
    query head, the ``top_k`` best blocks (ties: lower block), exact softmax attention over their tokens.
    ``q [B, Hq, D]``, ``K``/``V [B, Hkv, T, D]`` fp32, ``lens [B]`` -> ``[B, Hq, D]`` fp32."""
    out = torch.zeros(q.shape[0], q.shape[1], q.shape[2])
    for b in range(q.shape[0]):
        n = int(lens[b])
        nb = (n + block - 1) // block
        meta = skv_oracle.block_minmax_meta(K[b:b + 1, :, :n], block)
        sc = skv_oracle.quest_block_scores(q[b:b + 1], meta, scale)
        idx = skv_oracle.topk_blocks(sc, min(top_k, nb))
        out[b] = skv_oracle.attend_selected_blocks(q[b:b + 1], K[b:b + 1], V[b:b + 1], idx, block, scale,
                                                   lens[b:b + 1].to(torch.int32))[0]
    return out


def decode_step(weights: dict, cfg, tokens, k_hist, v_hist, seq_lens, layer_modes=None, quest_block: int = 64,
                quest_top_k: int = 8, v_bits: int = 8):
    """``weights``: fp32 full matrices (embed, lm_head, final_norm, layers[l][wq|wk|wv|wo|wg|wu|wd|n1|n2]);
    ``k_hist[l]``/``v_hist[l]``: ``[B, Hkv, Tmax, D]`` fp32 dequantised history; returns logits ``[B, vocab]``.
    ``layer_modes[l] == "quest"`` replaces the layer's dense attention by ``quest_attention`` (the per-layer schedule
    of the reference's ``sparse_layers``, benchmarks/llama_integration_benchmark.py:114-230).  ``v_bits=4``: the new
    token's value row is stored in 4 bits (mixed-precision pages) instead of FP8."""
    B = tokens.shape[0]
    D, Hq, Hkv = cfg.D, cfg.Hq, cfg.Hkv
    x = weights["embed"][tokens]
    pos = seq_lens.long()
    for l, w in enumerate(weights["layers"]):
        h = _rms(x, w["n1"], cfg.rms_eps)
        q = rope((h @ w["wq"]).view(B, Hq, D), pos, cfg.rope_theta)
        k = rope((h @ w["wk"]).view(B, Hkv, D), pos, cfg.rope_theta)
        v = (h @ w["wv"]).view(B, Hkv, D)
        kc, ks = skv_oracle.quantize_e4m3(k)
        if v_bits == 4:
            vq = skv_oracle.dequantize_int4(*skv_oracle.quantize_int4(v))
        else:
            vq = skv_oracle.dequantize(*skv_oracle.quantize_e4m3(v))
        kq = skv_oracle.dequantize(kc, ks)
        K, V = k_hist[l].clone(), v_hist[l].clone()
        for b in range(B):
            K[b, :, pos[b]] = kq[b]
            V[b, :, pos[b]] = vq[b]
        if layer_modes is not None and layer_modes[l] == "quest":
            a = quest_attention(q.half().float(), K, V, seq_lens + 1, quest_block, quest_top_k, 1.0 / math.sqrt(D))
        else:
            a = skv_oracle.dense_gqa_decode(q.half().float(), K.permute(0, 2, 1, 3), V.permute(0, 2, 1, 3),
                                            1.0 / math.sqrt(D), (seq_lens + 1).to(torch.int32))
        x = x + a.reshape(B, Hq * D) @ w["wo"]
        h = _rms(x, w["n2"], cfg.rms_eps)
        x = x + (torch.nn.functional.silu(h @ w["wg"]) * (h @ w["wu"])) @ w["wd"]
    return _rms(x, weights["final_norm"], cfg.rms_eps) @ weights["lm_head"]
