"""One decode step of a Llama-architecture model over a paged FP8 KV cache, tensor-parallel by KV head.

The reference measures this step by calling a Hugging Face model whose attention forward is
monkey-patched (benchmarks/llama_integration_benchmark.py:114-230, timed at :252-279); it is single-GPU
and needs the gated Llama-3.1-8B weights.  Here the step is written out directly so that it runs with
random weights of the same architecture on 1, 2, 4 or 8 GPUs:

    x -> [RMSNorm -> qkv GEMM -> RoPE -> quantise + append k,v to the paged cache -> paged decode
          attention (sm_100a kernel) -> o_proj GEMM -> all-reduce -> RMSNorm -> SwiGLU MLP -> all-reduce] x L
      -> RMSNorm -> lm_head

Rank r owns kv heads ``shard.kv_heads`` with their query heads (column-parallel q/k/v, gate, up;
row-parallel o_proj and down_proj), so the attention kernel reads only local pages and the only
collective is the sum all-reduce of the ``[batch, hidden]`` activations after o_proj and after down_proj
(NCCL over NVLink).  GEMMs are plain library GEMMs (cuBLAS through torch); the attention is this
package's kernel.  Weights are drawn per matrix from a generator seeded by (seed, layer, matrix) and
then sliced, so every tensor-parallel degree computes with the same full-model weights.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist
from torch import Tensor

from . import paged
from .sharding import HeadShard, shard_columns


@dataclass(frozen=True)
class ModelConfig:
    layers: int = 32
    hidden: int = 4096
    Hq: int = 32
    Hkv: int = 8
    D: int = 128
    mlp: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    init_std: float = 0.02


def _matrix(seed: int, layer: int, name: str, shape, device, dtype, std) -> Tensor:
    """Full (unsharded) weight matrix from a generator keyed by (seed, layer, name)."""
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + layer * 101 + sum(map(ord, name))) & 0x7FFFFFFF)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


def rms_norm(x: Tensor, w: Tensor, eps: float) -> Tensor:
    return torch.nn.functional.rms_norm(x, (x.shape[-1],), w, eps)


def rope(x: Tensor, pos: Tensor, theta: float) -> Tensor:
    """Plain rotary embedding (rotate-half form) of ``x [B, H, D]`` at integer positions ``pos [B]``."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
    xf = x.float()
    rot = torch.cat([-xf[..., D // 2:], xf[..., :D // 2]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


def quantize_rows_e4m3(x: Tensor):
    """Per-row FP8-E4M3 codes and fp32 scales (scale = amax / 448, 1 for a zero row) of ``x [..., D]``."""
    xf = x.float()
    amax = xf.abs().amax(-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    return (xf / scale[..., None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn), scale


def quantize_rows_int4(x: Tensor):
    """Packed 4-bit codes (nibble = code + 8, even channel low) and fp32 scales = amax / 7 of ``x [..., D]``."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 7.0, torch.ones_like(amax))
    u = (torch.round(xf / scale[..., None]).clamp_(-7.0, 7.0) + 8).to(torch.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).contiguous(), scale


class LayerCache:
    """Paged cache of one layer on one rank, page size 16: fused FP8 page records, or with ``v_bits=4`` mixed-precision
    records (FP8 keys, 4-bit values)."""

    def __init__(self, num_pages: int, n_kv: int, device, v_bits: int = 8):
        self.v_bits = v_bits
        rows = paged.MIXED_RECORD_ROWS if v_bits == 4 else paged.RECORD_ROWS
        self.buf = torch.zeros((num_pages, n_kv, rows, 128), dtype=torch.uint8, device=device)
        views = paged.mixed_views if v_bits == 4 else paged.fused_views
        self.k, self.v, self.ks, self.vs = views(self.buf, torch.float8_e4m3fn)

    def append(self, k: Tensor, v: Tensor, page_table: Tensor, seq_lens: Tensor) -> None:
        """Quantise the new token's ``k, v [B, n_kv, D]`` and store them at position ``seq_lens[b]``."""
        B = k.shape[0]
        lens = seq_lens.long()
        page = page_table[torch.arange(B, device=k.device), lens // 16].long()
        slot = lens % 16
        kc, ksc = quantize_rows_e4m3(k)
        vc, vsc = quantize_rows_int4(v) if self.v_bits == 4 else quantize_rows_e4m3(v)
        self.k.view(torch.uint8)[page, :, slot] = kc.view(torch.uint8)
        self.v.view(torch.uint8)[page, :, slot] = vc.view(torch.uint8)
        self.ks[page, :, slot] = ksc
        self.vs[page, :, slot] = vsc


AttentionFn = Callable[[Tensor, LayerCache, Tensor, Tensor, float, int], Tensor]


def kernel_attention(q: Tensor, cache: LayerCache, page_table: Tensor, seq_lens: Tensor, scale: float,
                     max_seq_len: int) -> Tensor:
    """The product path: paged FP8 decode attention on the sm_100a kernel (fp16 query in, fp16 out)."""
    from . import _C
    return _C.fused_gqa_paged(q.to(torch.float16).contiguous(), cache.k, cache.v, cache.ks, cache.vs, page_table,
                              seq_lens, scale, max_seq_len=max_seq_len, v_bits=cache.v_bits)


class DecodeModel:
    """The rank-local slice of the model and of every layer's cache."""

    def __init__(self, cfg: ModelConfig, shard: HeadShard, device, *, seed: int = 4, dtype=torch.bfloat16,
                 attention: AttentionFn = kernel_attention, group=None, layer_modes: list[str] | None = None,
                 quest_block: int = 64, quest_top_k: int = 8, skinny_gemm: bool = False, v_bits: int = 8):
        """``layer_modes``: per layer ``"dense"`` (attention over the whole cache) or ``"quest"`` (block-sparse: the
        ``quest_top_k`` blocks of ``quest_block`` tokens with the highest min/max upper-bound score per query head).
        The reference's layer sweep found sparse attention harmless in the first half of the layers only
        (results/llama_run_20260628_233732/layer_sweep.json:20-37; ``sparse_layers`` of its ``patch_attention``,
        benchmarks/llama_integration_benchmark.py:114-230): a schedule is this list."""
        self.cfg, self.shard, self.device, self.dtype = cfg, shard, torch.device(device), dtype
        self.attention, self.group = attention, group
        self.quest_block, self.quest_top_k = int(quest_block), int(quest_top_k)
        # True: the four projections of a layer run on this library's weight-streaming kernel (batches of up to 16
        # rows) instead of library GEMMs.  Off by default: measured on B200 the library GEMMs are faster at every
        # Llama-3-8B projection shape (graph replay, 16 rows: 79 us against 116 us per layer on one GPU).
        self.skinny_gemm = bool(skinny_gemm)
        # the dense attention kernel starts streaming the cache while the append kernel of the same layer is still running
        self.overlap_append = True
        # 4: the caches are mixed-precision page records (FP8 keys, 4-bit values: 200 instead of 264 bytes per token
        # and head)
        if v_bits not in (4, 8):
            raise ValueError("v_bits must be 4 or 8")
        self.v_bits = v_bits
        self.metas: list[Tensor | None] = []
        self.set_layer_modes(layer_modes)
        # the fused RoPE + quantise + append kernel needs fp16/bf16 activations on a CUDA device
        self.fused_glue = (self.device.type == "cuda" and dtype in (torch.float16, torch.bfloat16)
                           and attention is kernel_attention)
        self.fused_allreduce = False   # see enable_fused_allreduce
        D, hid = cfg.D, cfg.hidden
        qs = slice(shard.q_heads.start * D, shard.q_heads.stop * D)
        ks = slice(shard.kv_heads.start * D, shard.kv_heads.stop * D)
        ms = shard_columns(cfg.mlp, shard.world, shard.rank)
        ms = slice(ms.start, ms.stop)
        mk = lambda l, n, shp: _matrix(seed, l, n, shp, self.device, dtype, cfg.init_std)  # noqa: E731
        self.embed = mk(-1, "embed", (cfg.vocab, hid))
        # The output projection is split by vocabulary columns like the MLP (every rank streams 1/world of its 1 GB and
        # the logits are all-gathered) when the vocabulary divides evenly; otherwise every rank keeps the whole matrix.
        self.vocab_sharded = shard.world > 1 and cfg.vocab % shard.world == 0
        lm_head = mk(-2, "lm_head", (hid, cfg.vocab))
        if self.vocab_sharded:
            vs = shard_columns(cfg.vocab, shard.world, shard.rank)
            lm_head = lm_head[:, vs.start:vs.stop].contiguous()
        self.lm_head = lm_head
        self.final_norm = torch.ones(hid, device=self.device, dtype=dtype)
        self.layers = []
        for l in range(cfg.layers):
            wq, wk, wv = mk(l, "wq", (hid, cfg.Hq * D)), mk(l, "wk", (hid, cfg.Hkv * D)), mk(l, "wv", (hid, cfg.Hkv * D))
            wqkv = torch.cat([wq[:, qs], wk[:, ks], wv[:, ks]], 1).contiguous()
            del wq, wk, wv
            wo = mk(l, "wo", (cfg.Hq * D, hid))[qs].contiguous()
            wgu = torch.cat([mk(l, "wg", (hid, cfg.mlp))[:, ms], mk(l, "wu", (hid, cfg.mlp))[:, ms]], 1).contiguous()
            wd = mk(l, "wd", (cfg.mlp, hid))[ms].contiguous()
            self.layers.append(dict(wqkv=wqkv, wo=wo, wgu=wgu, wd=wd,
                                    n1=torch.ones(hid, device=self.device, dtype=dtype),
                                    n2=torch.ones(hid, device=self.device, dtype=dtype)))
        self.caches: list[LayerCache] = []
        self.page_table: Tensor | None = None
        self.seq_lens: Tensor | None = None
        self.max_seq_len = 0

    # ------------------------------------------------------------------ per-layer sparsity schedule
    def set_layer_modes(self, layer_modes: list[str] | None) -> None:
        """Choose dense or Quest block-sparse attention per layer; builds the block metadata of layers that turn sparse."""
        modes = list(layer_modes) if layer_modes is not None else ["dense"] * self.cfg.layers
        if len(modes) != self.cfg.layers or any(m not in ("dense", "quest") for m in modes):
            raise ValueError("layer_modes must name 'dense' or 'quest' for every layer")
        if self.v_bits == 4 and "quest" in modes and self.quest_block * self.quest_top_k > 512:
            raise ValueError("block-sparse layers over 4-bit values gather at most 512 tokens (quest_block * quest_top_k)")
        self.layer_modes = modes
        if getattr(self, "caches", None):
            for l, m in enumerate(modes):   # a dense layer's appends do not maintain metadata: drop what would go stale
                if m == "dense" and l < len(self.metas):
                    self.metas[l] = None
            self._build_missing_metas()

    def _layer_kv(self, cache: "LayerCache", lens: Tensor):
        return paged.PagedKV(cache.k, cache.v, cache.ks, cache.vs, self.page_table, lens, lens.numel(), v_bits=cache.v_bits)

    def _build_missing_metas(self) -> None:
        if len(self.metas) != len(self.caches):
            self.metas = [None] * len(self.caches)
        for l, (mode, cache) in enumerate(zip(self.layer_modes, self.caches)):
            if mode == "quest" and self.metas[l] is None:
                self.metas[l] = paged.build_block_meta(self._layer_kv(cache, self.seq_lens), self.quest_block,
                                                       max_seq_len=self.max_seq_len)

    def _quest_attention(self, q: Tensor, l: int, new_lens: Tensor, scale: float, meta_is_current: bool) -> Tensor:
        """Block-sparse attention of layer ``l`` for fp16 ``q [B, n_q, D]`` over the cache holding ``new_lens`` tokens."""
        kv = self._layer_kv(self.caches[l], new_lens)
        if not meta_is_current:   # the eager append of the fp32 test path does not touch the metadata
            self.metas[l] = paged.build_block_meta(kv, self.quest_block, max_seq_len=self.max_seq_len)
        return paged.quest_sparse_decode(q, kv, self.metas[l], scale, self.quest_block, self.quest_top_k,
                                         max_seq_len=self.max_seq_len)

    # ------------------------------------------------------------------ cache set-up
    def init_cache(self, seq_lens: Tensor, *, fill: str = "normal", seed: int = 4, extra_tokens: int = 64) -> None:
        """Allocate every layer's pages for sequences of the given lengths and pre-fill them.

        No prefill pass is run (only the decode step is the workload): ``fill="normal"`` writes N(0,1)
        keys/values quantised row by row to FP8; ``fill="random_codes"`` writes uniformly random FP8 codes with
        scales near 0.008 (values within about +-4), which is much faster to generate for a 70 GB cache and
        costs the kernels the same time.  Pages are assigned to (sequence, logical page) by a seeded permutation.
        """
        cfg, dev = self.cfg, self.device
        B = seq_lens.numel()
        cap = (seq_lens.max().item() + extra_tokens + 15) // 16
        pages_per_seq = [(int(n) + extra_tokens + 15) // 16 for n in seq_lens.tolist()]
        total = sum(pages_per_seq)
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(total, generator=g)
        table = torch.zeros((B, cap), dtype=torch.int32)
        o = 0
        for b, n in enumerate(pages_per_seq):
            table[b, :n] = perm[o:o + n].to(torch.int32)
            o += n
        self.page_table = table.to(dev)
        self.seq_lens = seq_lens.to(device=dev, dtype=torch.int32).clone()
        self.max_seq_len = cap * 16
        self.caches = []
        gd = torch.Generator(device=dev)
        for l in range(cfg.layers):
            c = LayerCache(total, self.shard.n_kv, dev, self.v_bits)
            for i, head in enumerate(self.shard.kv_heads):  # keyed by the GLOBAL head: same bytes at every TP degree
                gd.manual_seed((seed * 7919 + l * 131 + head) & 0x7FFFFFFF)
                if fill == "normal":
                    for dst, dsc, quant in ((c.k, c.ks, quantize_rows_e4m3),
                                            (c.v, c.vs, quantize_rows_int4 if self.v_bits == 4 else quantize_rows_e4m3)):
                        codes, sc = quant(torch.randn((total, 16, 128), generator=gd, device=dev))
                        dst.view(torch.uint8)[:, i].copy_(codes.view(torch.uint8))
                        dsc[:, i].copy_(sc)
                elif fill == "random_codes":
                    codes = torch.randint(0, 256, (total, c.buf.shape[2], 128), generator=gd, device=dev, dtype=torch.uint8)
                    codes = torch.where((codes & 0x7F) == 0x7F, codes & 0xFE, codes)  # keep clear of the NaN patterns
                    c.buf[:, i].copy_(codes)
                    del codes
                    c.ks[:, i].copy_(torch.rand((total, 16), generator=gd, device=dev) * 0.004 + 0.006)
                    # (4-bit values span -8..7 where FP8 codes span +-448: a scale that keeps the values within about +-4)
                    c.vs[:, i].copy_((torch.rand((total, 16), generator=gd, device=dev) * 0.004 + 0.006) * (64.0 if self.v_bits == 4 else 1.0))
                elif fill != "zeros":
                    raise ValueError(f"unknown fill {fill!r}")
            self.caches.append(c)
        self.metas = [None] * cfg.layers
        self._build_missing_metas()

    # ------------------------------------------------------------------ the step
    def _all_reduce(self, x: Tensor) -> Tensor:
        if self.shard.world > 1:
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.group)
        return x

    def _step_fused_allreduce(self, x: Tensor, pos: Tensor, new_lens: Tensor, scale: float) -> Tensor:
        """The layer loop with both all-reduces fused into the RMSNorm kernels that follow them (no NCCL call).

        o_proj writes its partial into buffer 0 and down_proj into buffer 1 of ``self.arn``; the kernel that
        normalises for the next GEMM sums the peers' partials over NVLink first.
        """
        from . import _C, glue
        cfg, sh, arn = self.cfg, self.shard, self.arn
        D, B = cfg.D, x.shape[0]
        h = glue.residual_rmsnorm(x, None, self.layers[0]["n1"], cfg.rms_eps)
        for li, (w, cache) in enumerate(zip(self.layers, self.caches)):
            qkv = self._mm(h, w["wqkv"])
            a = self._fused_attention(li, qkv, cache, pos, new_lens, scale, x.dtype)
            self._mm(a.view(B, sh.n_q * D), w["wo"], out=arn.partial(0))
            h = arn.reduce_norm(0, x, w["n2"], cfg.rms_eps)
            self._mm(glue.silu_mul(self._mm(h, w["wgu"])), w["wd"], out=arn.partial(1))
            nxt = self.layers[li + 1]["n1"] if li + 1 < len(self.layers) else self.final_norm
            h = arn.reduce_norm(1, x, nxt, cfg.rms_eps)
        self.seq_lens.add_(1)
        return self._logits(h)

    def _logits(self, h: Tensor) -> Tensor:
        """``h [B, hidden]`` -> logits ``[B, vocab]`` (all-gather of the ranks' column slices when the head is sharded)."""
        local = h @ self.lm_head
        if not self.vocab_sharded:
            return local
        return self._all_gather_columns(local)

    def _all_gather_columns(self, local: Tensor) -> Tensor:
        world = self.shard.world
        B, cols = local.shape
        parts = torch.empty((world * B, cols), dtype=local.dtype, device=local.device)   # rank r's rows at [r*B, (r+1)*B)
        dist.all_gather_into_tensor(parts, local.contiguous(), group=self.group)
        return parts.view(world, B, cols).permute(1, 0, 2).reshape(B, world * cols)

    def _mm(self, x: Tensor, w: Tensor, out: Tensor | None = None) -> Tensor:
        """``x @ w`` of the fused-glue path: the weight-streaming kernel where it applies, else the library GEMM."""
        from . import glue
        if self.skinny_gemm and glue.skinny_gemm_supported(x.shape[0], w.shape[0], w.shape[1]) and x.is_contiguous():
            return glue.skinny_gemm(x, w, out=out)
        return torch.matmul(x, w, out=out) if out is not None else x @ w

    def _fused_attention(self, li: int, qkv: Tensor, cache: "LayerCache", pos: Tensor, new_lens: Tensor, scale: float,
                         dtype) -> Tensor:
        """RoPE + quantise + append (one launch, which also keeps a sparse layer's block metadata current), then the
        layer's attention: dense over the whole paged cache, or Quest block-sparse; ``[B, n_q, D]`` in ``dtype``."""
        from . import _C
        sh, D, B = self.shard, self.cfg.D, qkv.shape[0]
        sparse = self.layer_modes[li] == "quest"
        q = paged.rope_quant_append(qkv, self._layer_kv(cache, pos), sh.n_q, self.cfg.rope_theta,
                                    meta=self.metas[li] if sparse else None, block_size=self.quest_block)
        if sparse:
            return self._quest_attention(q, li, new_lens, scale, meta_is_current=True).to(dtype)
        a = torch.empty((B, sh.n_q, D), dtype=dtype, device=qkv.device)
        # the append kernel above is the launch right before this one and wrote only q and position new_lens - 1
        _C.fused_gqa_paged(q, cache.k, cache.v, cache.ks, cache.vs, self.page_table, new_lens, scale,
                           max_seq_len=self.max_seq_len, out=a, v_bits=cache.v_bits, after_append=self.overlap_append)
        return a

    def enable_fused_allreduce(self, batch: int, protocol: str | None = None) -> None:
        """Replace the two NCCL all-reduces per layer by the fused peer-memory kernel (CUDA, world > 1, fixed batch).
        ``protocol``: ``"pull"`` (flag, then loads from the peers; the default) or ``"push"`` (every rank writes its
        tagged partial into the peers' receive regions: measured faster on 2 GPUs, 6.8 against 7.7 us per call, and
        slower from 4 GPUs up, where the doubled NVLink bytes of the tagged words cost more than the saved traversal);
        ``SKV_ALLREDUCE_PROTOCOL`` in the environment overrides the default."""
        from . import glue
        if not self.fused_glue or self.shard.world == 1:
            raise RuntimeError("the fused all-reduce needs the CUDA glue path and more than one rank")
        if protocol is None:
            protocol = os.environ.get("SKV_ALLREDUCE_PROTOCOL") or "pull"
        self.arn = glue.AllReduceNorm(batch, self.cfg.hidden, self.dtype, self.device, self.group, protocol=protocol)
        self.fused_allreduce = True

    def step(self, tokens: Tensor) -> Tensor:
        """Decode one token per sequence: ``tokens [B]`` int64 -> logits ``[B, vocab]``; advances ``seq_lens``."""
        cfg, sh = self.cfg, self.shard
        D = cfg.D
        B = tokens.shape[0]
        scale = 1.0 / math.sqrt(D)
        x = self.embed[tokens]
        pos = self.seq_lens
        new_lens = self.seq_lens + 1
        if self.fused_glue:
            # Per layer: residual+RMSNorm, qkv GEMM, RoPE+quantise+append, attention (writing the model dtype),
            # o_proj GEMM, residual+RMSNorm, gate/up GEMM, SiLU*up, down GEMM -- four of our launches and four GEMMs.
            # The residual stream x is updated in place; `delta` is the MLP output still to be added to it.
            from . import _C, glue
            if self.fused_allreduce:
                return self._step_fused_allreduce(x, pos, new_lens, scale)
            delta = None
            for li, (w, cache) in enumerate(zip(self.layers, self.caches)):
                h = glue.residual_rmsnorm(x, delta, w["n1"], cfg.rms_eps)
                qkv = self._mm(h, w["wqkv"])
                a = self._fused_attention(li, qkv, cache, pos, new_lens, scale, x.dtype)
                o = self._all_reduce(self._mm(a.view(B, sh.n_q * D), w["wo"]))
                h = glue.residual_rmsnorm(x, o, w["n2"], cfg.rms_eps)
                delta = self._all_reduce(self._mm(glue.silu_mul(self._mm(h, w["wgu"])), w["wd"]))
            self.seq_lens.add_(1)
            return self._logits(glue.residual_rmsnorm(x, delta, self.final_norm, cfg.rms_eps))
        for li, (w, cache) in enumerate(zip(self.layers, self.caches)):
            h = rms_norm(x, w["n1"], cfg.rms_eps)
            qkv = h @ w["wqkv"]
            q = qkv[:, :sh.n_q * D].view(B, sh.n_q, D)
            k = qkv[:, sh.n_q * D:(sh.n_q + sh.n_kv) * D].view(B, sh.n_kv, D)
            v = qkv[:, (sh.n_q + sh.n_kv) * D:].view(B, sh.n_kv, D)
            q, k = rope(q, pos, cfg.rope_theta), rope(k, pos, cfg.rope_theta)
            cache.append(k, v, self.page_table, pos)
            if self.layer_modes[li] == "quest":
                a = self._quest_attention(q.to(torch.float16).contiguous(), li, new_lens, scale, meta_is_current=False)
            else:
                a = self.attention(q, cache, self.page_table, new_lens, scale, self.max_seq_len)
            o = a.to(x.dtype).reshape(B, sh.n_q * D) @ w["wo"]
            x = x + self._all_reduce(o)
            h = rms_norm(x, w["n2"], cfg.rms_eps)
            gu = h @ w["wgu"]
            half = gu.shape[1] // 2
            act = torch.nn.functional.silu(gu[:, :half]) * gu[:, half:]
            x = x + self._all_reduce(act @ w["wd"])
        self.seq_lens.add_(1)
        return self._logits(rms_norm(x, self.final_norm, cfg.rms_eps))
