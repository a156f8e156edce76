"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Everything is generated with the CPU generator so that the CPU oracle and the
GPU path see bit-identical inputs; callers move tensors to the device.
"""
from __future__ import annotations

import math

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def token_sparse_config1(seed: int = 0):
    """B=1, H=8, D=64, context 1024, single query token; Q/K/V ~ N(0,1), fp32.

    Uses the global CPU RNG stream of ``torch.manual_seed(seed)`` (the call the
    reference's own scripts make), so the golden fixtures stay reproducible.
    """
    torch.manual_seed(seed)
    Q = torch.randn(1, 8, 1, 64)
    K = torch.randn(1, 8, 1024, 64)
    V = torch.randn(1, 8, 1024, 64)
    return Q, K, V


def dense_gqa(N: int, B: int = 1, Hq: int = 32, Hkv: int = 8, D: int = 128, seed: int = 1):
    """Llama-3.1-8B layer shape: Q [B,Hq,D], K/V [B,N,Hkv,D] fp16, values N(0,1)/sqrt(D); scale 1/sqrt(D)."""
    g = _gen(seed)
    inv = 1.0 / math.sqrt(D)
    Q = (torch.randn(B, Hq, D, generator=g) * inv).half()
    K = (torch.randn(B, N, Hkv, D, generator=g) * inv).half()
    V = (torch.randn(B, N, Hkv, D, generator=g) * inv).half()
    return Q, K, V, inv


def eviction(B: int = 4, H: int = 8, T: int = 32768, D: int = 128, rounds: int = 32, seed: int = 2):
    """fp16 cache [B,H,T,D] ~ N(0,1) with 2 % of channels scaled x8, fp32 importance scores.

    Scores are the sum over ``rounds`` decode steps of softmax(N(0,2) logits).
    """
    g = _gen(seed)
    n_out = max(1, round(0.02 * D))
    K = torch.randn(B, H, T, D, generator=g)
    V = torch.randn(B, H, T, D, generator=g)
    K[..., torch.randperm(D, generator=g)[:n_out]] *= 8.0
    V[..., torch.randperm(D, generator=g)[:n_out]] *= 8.0
    scores = torch.zeros(B, H, T)
    for _ in range(rounds):
        scores += torch.softmax(2.0 * torch.randn(B, H, T, generator=g), dim=-1)
    return K.half(), V.half(), scores


def planted_block_cache(B: int, Hq: int, Hkv: int, T: int, D: int = 128, block_size: int = 64, planted: int = 8,
                        cosine: float = 0.9, seed: int = 3):
    """Q [B,Hq,D], K/V [B,Hkv,T,D] ~ N(0,1) (fp16) with `planted` high-affinity blocks per (b, kv-head).

    Every key of a planted block is re-aimed at the normalised sum of the group's queries with the given
    cosine, keeping its norm.  Returns (Q, K, V, planted_block_ids [B,Hkv,planted]).
    """
    g = _gen(seed)
    G = Hq // Hkv
    nb = T // block_size
    Q = torch.randn(B, Hq, D, generator=g)
    K = torch.randn(B, Hkv, T, D, generator=g)
    V = torch.randn(B, Hkv, T, D, generator=g)
    ids = torch.empty(B, Hkv, planted, dtype=torch.long)
    sin = math.sqrt(1.0 - cosine * cosine)
    for b in range(B):
        for h in range(Hkv):
            u = Q[b, h * G:(h + 1) * G].sum(0)
            u = u / u.norm()
            blocks = torch.randperm(nb, generator=g)[:planted]
            ids[b, h] = blocks.sort().values
            for j in blocks.tolist():
                k = K[b, h, j * block_size:(j + 1) * block_size]
                norm = k.norm(dim=-1, keepdim=True)
                orth = k - (k @ u)[:, None] * u
                orth = orth / orth.norm(dim=-1, keepdim=True)
                K[b, h, j * block_size:(j + 1) * block_size] = norm * (cosine * u + sin * orth)
    return Q.half(), K.half(), V.half(), ids
