"""CPU oracle for the long-context decode path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module: it is the checker used by
``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of
``bench.py``.  Every function restates, in fp32 torch on the CPU, the arithmetic
of one reference function (cited by path:line inside the reference project) or,
where the reference has no implementation, the rule fixed by this project's
specification (marked "no reference counterpart").

Pinning: the reference's tests hold no golden values for this path, so the
restatements of ``_reference_sparse_attention`` and ``_reference_eviction`` are
pinned against outputs of the reference's own Python functions, generated once
by ``tests/golden/make_golden.py`` and committed under ``tests/golden/``.  The
pieces without a reference counterpart (scaled INT8 / FP8 quantisation, paging,
min/max block metadata, the recent-token window, the split-KV combine) are
"parity unpinned": their only anchor is the written rule in each docstring.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

E4M3_MAX = 448.0
INT8_MAX = 127.0


# --------------------------------------------------------------------------- dense GQA decode
def dense_gqa_decode(Q: Tensor, K: Tensor, V: Tensor, scale: float, seq_lens: Tensor | None = None) -> Tensor:
    """fp32 ``softmax(scale * q K^T) V`` per query head, kv head ``hq // (Hq // Hkv)``.

    Restates the reference's own validation of ``fused_gqa``: SDPA over
    ``repeat_kv``-expanded K/V (benchmarks/llama_integration_benchmark.py:464-471) and the
    kernel's head mapping (csrc/kernels/gqa_decode.cu:96-97).
    Q ``[B,Hq,D]``, K/V ``[B,N,Hkv,D]`` -> ``[B,Hq,D]`` fp32.
    """
    B, Hq, D = Q.shape
    N, Hkv = K.shape[1], K.shape[2]
    G = Hq // Hkv
    q = Q.float().reshape(B, Hkv, G, D)
    k = K.float().permute(0, 2, 1, 3)  # [B,Hkv,N,D]
    v = V.float().permute(0, 2, 1, 3)
    s = torch.matmul(q, k.transpose(-1, -2)) * float(scale)  # [B,Hkv,G,N]
    if seq_lens is not None:
        pos = torch.arange(N).view(1, 1, 1, N)
        s = s.masked_fill(pos >= seq_lens.view(B, 1, 1, 1).long(), float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)  # an empty sequence yields zeros
    return torch.matmul(p, v).reshape(B, Hq, D)


def attention_mass(Q: Tensor, K: Tensor, scale: float, seq_lens: Tensor | None = None) -> Tensor:
    """Attention probability of every cached token, summed over the query heads of its kv-head: ``[B,Hkv,N]`` fp32.

    The per-token importance an eviction policy accumulates over decode steps; it is what the reference's
    ``fused_kv_evict`` expects as ``scores`` (sparse_kv/eviction.py:12-22; the reference has no code that
    produces it).  Tokens past ``seq_lens`` get zero.
    """
    B, Hq, D = Q.shape
    N, Hkv = K.shape[1], K.shape[2]
    G = Hq // Hkv
    q = Q.float().reshape(B, Hkv, G, D)
    k = K.float().permute(0, 2, 1, 3)
    s = torch.matmul(q, k.transpose(-1, -2)) * float(scale)
    if seq_lens is not None:
        pos = torch.arange(N).view(1, 1, 1, N)
        s = s.masked_fill(pos >= seq_lens.view(B, 1, 1, 1).long(), float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    return p.sum(dim=2)


def combine_split_partials(m: Tensor, l: Tensor, o: Tensor) -> Tensor:
    """Log-sum-exp merge of per-split partial results (no reference counterpart).

    ``m``/``l`` ``[S, ...]`` running max and sum, ``o`` ``[S, ..., D]`` un-normalised
    outputs relative to ``m``:  ``M = max m_i``, ``L = sum l_i e^{m_i-M}``,
    ``O = sum o_i e^{m_i-M} / L``.
    """
    M = m.max(dim=0).values
    w = torch.exp(m - M)
    L = (l * w).sum(0)
    return (o * w.unsqueeze(-1)).sum(0) / L.unsqueeze(-1)


# --------------------------------------------------------------------------- token-sparse decode
def token_sparse_attention(Q: Tensor, K: Tensor, V: Tensor, top_k: int, sink_tokens: int) -> Tensor:
    """Attention restricted to the ``top_k`` highest-scoring keys plus the first ``sink_tokens``.

    Restates ``_reference_sparse_attention`` (sparse_kv/attention.py:25-38):
    scores ``q.k * D^-0.5``; every position outside (top-k set U sink prefix) is
    excluded; softmax over what remains; weighted sum of V.
    Q ``[B,H,S,D]``, K/V ``[B,H,T,D]`` -> ``[B,H,S,D]`` in Q's dtype.
    """
    D = Q.shape[-1]
    T = K.shape[2]
    s = torch.matmul(Q, K.transpose(-1, -2)) * (D ** -0.5)  # [B,H,S,T]
    keep = torch.zeros(s.shape, dtype=torch.bool)
    top = torch.topk(s, min(top_k, T), dim=-1).indices
    keep.scatter_(-1, top, True)
    if sink_tokens > 0:
        keep[..., :sink_tokens] = True
    s = torch.where(keep, s, torch.full_like(s, float("-inf")))
    return torch.matmul(torch.softmax(s, dim=-1), V)


def token_topk_sets(Q: Tensor, K: Tensor, top_k: int) -> Tensor:
    """Sorted indices of the ``top_k`` best-scoring keys per (b, h) for a one-token query."""
    s = torch.matmul(Q.float(), K.float().transpose(-1, -2))[:, :, 0, :]
    return torch.topk(s, min(top_k, K.shape[2]), dim=-1).indices.sort(-1).values


# --------------------------------------------------------------------------- block-sparse decode (mean rule)
def block_mean_scores(Q: Tensor, K: Tensor, block_size: int) -> Tensor:
    """``scale * mean_{t in block}(q . k_t)``; the ragged last block divides by its own count.

    Restates step 1 of ``block_sparse_attn_kernel`` (csrc/kernels/sparse_attention.cu:51-78)
    and of ``sparse_attention_reference`` (jax_ref/sparse_attention_pallas.py:85-104).
    Q ``[B,H,1,D]``, K ``[B,H,T,D]`` -> ``[B,H,nb]`` fp32.
    """
    B, H, T, D = K.shape
    nb = (T + block_size - 1) // block_size
    dots = torch.matmul(K.float(), Q.float()[:, :, 0, :, None])[..., 0] / math.sqrt(D)  # [B,H,T]
    pad = nb * block_size - T
    if pad:
        dots = torch.nn.functional.pad(dots, (0, pad))
    sums = dots.view(B, H, nb, block_size).sum(-1)
    counts = torch.full((nb,), float(block_size))
    if pad:
        counts[-1] = block_size - pad
    return sums / counts


def block_sparse_mean_attention(Q: Tensor, K: Tensor, V: Tensor, block_size: int, top_k_blocks: int):
    """The reference's block-sparse decode: softmax over the k best block scores, block-mean values.

    Restates ``block_sparse_attn_kernel`` steps 2-4 (csrc/kernels/sparse_attention.cu:88-169) and
    ``sparse_attention_reference`` (jax_ref/sparse_attention_pallas.py:106-133):
    ``w = softmax(top-k block scores)``, ``out = sum_j w_j * mean_{t in block j} v_t``.
    Returns ``(out [B,H,1,D] fp32, sorted block ids [B,H,k])``; ties go to the lower block id.
    """
    B, H, T, D = K.shape
    nb = (T + block_size - 1) // block_size
    k = min(top_k_blocks, nb)
    sc = block_mean_scores(Q, K, block_size)
    top_v, top_i = torch.topk(sc, k, dim=-1)
    w = torch.softmax(top_v, dim=-1)  # [B,H,k]
    pad = nb * block_size - T
    v = V.float()
    if pad:
        v = torch.nn.functional.pad(v, (0, 0, 0, pad))
    counts = torch.full((nb,), float(block_size))
    if pad:
        counts[-1] = block_size - pad
    vmean = v.view(B, H, nb, block_size, D).sum(3) / counts.view(1, 1, nb, 1)
    sel = torch.gather(vmean, 2, top_i.unsqueeze(-1).expand(-1, -1, -1, D))
    out = (sel * w.unsqueeze(-1)).sum(2, keepdim=True)
    return out, top_i.sort(-1).values


# --------------------------------------------------------------------------- eviction: which tokens stay
def eviction_keep_indices(scores: Tensor, budget: int, recent: int = 0) -> Tensor:
    """Ascending positions of the tokens that survive eviction, ``[B,H,keep]`` int64.

    The ``budget`` highest-scoring tokens are found the way ``_reference_eviction`` does
    (sparse_kv/eviction.py:37, ``attn_scores.topk(top_k)``).  The last ``recent``
    positions are always kept (no reference counterpart): they are given score
    +inf so the same ``topk`` returns them, ``keep = budget + recent``.  The
    result is sorted by position because the compacted cache keeps token order.
    """
    s = scores.float().clone()
    T = s.shape[-1]
    recent = min(recent, T)
    if recent:
        s[..., T - recent:] = float("inf")
    keep = min(budget + recent, T)
    return torch.topk(s, keep, dim=-1).indices.sort(-1).values


def evict_gather(K: Tensor, V: Tensor, idx: Tensor):
    """Rows of K/V ``[B,H,T,D]`` at ``idx [B,H,keep]`` (sparse_kv/eviction.py:38-40)."""
    ix = idx.unsqueeze(-1).expand(-1, -1, -1, K.shape[-1])
    return K.gather(2, ix), V.gather(2, ix)


# --------------------------------------------------------------------------- quantisation (no reference counterpart)
def quantize_int8(x: Tensor):
    """Symmetric INT8 per row of D channels.

    ``amax = max|x|`` in fp32; ``scale = amax / 127`` (1.0 when the row is all zero);
    ``code = clamp(round_half_even(x / scale), -127, 127)``.  Returns (int8 codes, fp32 scales[...]).
    The reference's own "INT8" is an unscaled cast (sparse_kv/eviction.py:41-43) and its CUDA
    launcher rejects it (csrc/kernels/kv_evict_quant.cu:294); this rule replaces both.
    """
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / INT8_MAX, torch.ones_like(amax))
    q = torch.round(xf / scale.unsqueeze(-1)).clamp_(-INT8_MAX, INT8_MAX)
    return q.to(torch.int8), scale


def quantize_e4m3(x: Tensor):
    """FP8-E4M3 (finite-only, max 448) per row: ``scale = amax / 448``, RNE conversion of ``x / scale``."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    y = (xf / scale.unsqueeze(-1)).clamp_(-E4M3_MAX, E4M3_MAX)
    return y.to(torch.float8_e4m3fn), scale


INT4_MAX = 7.0


def quantize_int4(x: Tensor):
    """Symmetric 4-bit codes per row of D channels, for the V half of mixed-precision pages.

    ``scale = amax / 7`` (1.0 for a zero row); ``q = clamp(round_half_even(x / scale), -7, 7)``; the stored nibble is
    ``q + 8`` (1..15) and byte ``j`` of a row holds channel ``2j`` in its low and channel ``2j+1`` in its high nibble.
    Returns (uint8 [..., D/2] packed codes, fp32 scales[...]).  No reference counterpart.
    """
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / INT4_MAX, torch.ones_like(amax))
    q = torch.round(xf / scale.unsqueeze(-1)).clamp_(-INT4_MAX, INT4_MAX)
    u = (q + 8).to(torch.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).contiguous(), scale


def dequantize_int4(packed: Tensor, scale: Tensor) -> Tensor:
    """fp32 values of 4-bit codes packed by :func:`quantize_int4`."""
    lo = (packed & 0x0F).to(torch.int16) - 8
    hi = (packed >> 4).to(torch.int16) - 8
    q = torch.stack((lo, hi), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    return q.float() * scale.float().unsqueeze(-1)


def dequantize(codes: Tensor, scale: Tensor) -> Tensor:
    return codes.float() * scale.unsqueeze(-1)


def e4m3_code_distance(a: Tensor, b: Tensor) -> Tensor:
    """Distance in code steps between two e4m3 tensors (sign-magnitude bytes mapped to a line)."""
    def line(t):
        u = t.view(torch.uint8).to(torch.int16)
        mag = u & 0x7F
        return torch.where((u & 0x80) != 0, -mag, mag)
    return (line(a) - line(b)).abs()


# --------------------------------------------------------------------------- paged cache + block metadata (no reference counterpart)
def build_paged_cache(codes: Tensor, scales: Tensor, page_size: int, perm: Tensor):
    """Scatter a ``[B,Hkv,T,D]`` quantised cache into a page pool.

    Pool ``[num_pages, Hkv, page_size, D]`` codes and ``[num_pages, Hkv, page_size]`` scales;
    ``page_table[b, i] = perm[b * pages_per_seq + i]`` names the physical page of
    logical page ``i`` of sequence ``b``.  T must be a multiple of ``page_size`` here.
    """
    B, H, T, D = codes.shape
    pps = T // page_size
    table = perm[: B * pps].view(B, pps).to(torch.int32)
    num_pages = int(perm.numel())
    pool = torch.zeros((num_pages, H, page_size, D), dtype=codes.dtype)
    spool = torch.zeros((num_pages, H, page_size), dtype=torch.float32)
    src = codes.view(B, H, pps, page_size, D).permute(0, 2, 1, 3, 4).reshape(B * pps, H, page_size, D)
    ssrc = scales.view(B, H, pps, page_size).permute(0, 2, 1, 3).reshape(B * pps, H, page_size)
    pool[table.view(-1).long()] = src
    spool[table.view(-1).long()] = ssrc
    return pool, spool, table


def block_minmax_meta(Kdeq: Tensor, block_size: int) -> Tensor:
    """Channel-wise min and max of the dequantised keys of every block: ``[B,Hkv,nb,2,D]`` fp16."""
    B, H, T, D = Kdeq.shape
    nb = (T + block_size - 1) // block_size
    pad = nb * block_size - T
    lo_src, hi_src = Kdeq.float(), Kdeq.float()
    if pad:
        lo_src = torch.nn.functional.pad(lo_src, (0, 0, 0, pad), value=float("inf"))
        hi_src = torch.nn.functional.pad(hi_src, (0, 0, 0, pad), value=float("-inf"))
    lo = lo_src.view(B, H, nb, block_size, D).amin(3)
    hi = hi_src.view(B, H, nb, block_size, D).amax(3)
    return torch.stack([lo, hi], dim=3).to(torch.float16)


def quest_block_scores(Q: Tensor, meta: Tensor, scale: float) -> Tensor:
    """Upper bound of ``scale * q.k`` over a block: ``scale * sum_d max(q_d*min_d, q_d*max_d)``.

    Q ``[B,Hq,D]``, meta ``[B,Hkv,nb,2,D]`` -> ``[B,Hq,nb]`` fp32, one score per *query* head.
    """
    B, Hq, D = Q.shape
    Hkv = meta.shape[1]
    G = Hq // Hkv
    q = Q.float().view(B, Hkv, G, 1, D)
    lo = meta[:, :, :, 0].float().unsqueeze(2)
    hi = meta[:, :, :, 1].float().unsqueeze(2)
    return (torch.maximum(q * lo, q * hi).sum(-1) * float(scale)).reshape(B, Hq, -1)


def topk_blocks(scores: Tensor, k: int) -> Tensor:
    """Sorted ids of the k best blocks; equal scores resolve to the lower id."""
    nb = scores.shape[-1]
    k = min(k, nb)
    order = torch.argsort(scores, dim=-1, descending=True, stable=True)
    return order[..., :k].sort(-1).values


def attend_selected_blocks(Q: Tensor, Kdeq: Tensor, Vdeq: Tensor, blocks: Tensor, block_size: int,
                           scale: float, seq_lens: Tensor | None = None) -> Tensor:
    """Exact softmax attention over the tokens of the selected blocks only.

    Q ``[B,Hq,D]``, K/V dequantised ``[B,Hkv,T,D]``, ``blocks [B,Hq,k]`` -> ``[B,Hq,D]`` fp32.
    """
    B, Hq, D = Q.shape
    Hkv, T = Kdeq.shape[1], Kdeq.shape[2]
    G = Hq // Hkv
    out = torch.zeros(B, Hq, D)
    for b in range(B):
        n = T if seq_lens is None else int(seq_lens[b])
        for hq in range(Hq):
            tok = (blocks[b, hq].long().view(-1, 1) * block_size + torch.arange(block_size).view(1, -1)).view(-1)
            tok = tok[(tok < n) & (blocks[b, hq].long().repeat_interleave(block_size) >= 0)]
            kk = Kdeq[b, hq // G, tok].float()
            vv = Vdeq[b, hq // G, tok].float()
            s = (kk @ Q[b, hq].float()) * float(scale)
            out[b, hq] = torch.softmax(s, 0) @ vv
    return out
