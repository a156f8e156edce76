"""Paged 8-bit KV cache: container, block metadata and Quest-style sparse decode.

No counterpart in the reference, whose caches are unpaged fp16 tensors; the layout is
code pools ``[num_pages, Hkv, page_size, D]`` (int8 or float8_e4m3fn), fp32 scale pools
``[num_pages, Hkv, page_size]`` and an int32 ``page_table [B, max_pages]``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

from . import _C, _lib, _workspace


@dataclass
class PagedKV:
    k_pool: Tensor
    v_pool: Tensor
    k_scale: Tensor
    v_scale: Tensor
    page_table: Tensor | None   # int32 [B, max_pages]; None: sequence b owns pages b*max_pages ...
    seq_lens: Tensor | None     # int32 [B]
    batch: int
    v_bits: int = 8             # 4: mixed-precision page records, v_pool is uint8 [num_pages, Hkv, 16, 64] (see mixed_views)

    @property
    def page_size(self) -> int:
        return self.k_pool.shape[2]

    @property
    def max_pages(self) -> int:
        return self.page_table.shape[1] if self.page_table is not None else self.k_pool.shape[0] // self.batch

    @property
    def capacity(self) -> int:
        return self.max_pages * self.page_size

    @classmethod
    def from_fused(cls, buf: Tensor, code_dtype: torch.dtype, page_table: Tensor | None, seq_lens: Tensor | None,
                   batch: int) -> "PagedKV":
        """Cache whose pools are views of one fused page-record buffer (see ``fused_views``)."""
        k, v, ks, vs = fused_views(buf, code_dtype)
        return cls(k, v, ks, vs, page_table, seq_lens, batch)

    @classmethod
    def from_mixed(cls, buf: Tensor, code_dtype: torch.dtype, page_table: Tensor | None, seq_lens: Tensor | None,
                   batch: int) -> "PagedKV":
        """Cache of mixed-precision page records: 8-bit K, 4-bit V (see ``mixed_views``)."""
        k, v, ks, vs = mixed_views(buf, code_dtype)
        return cls(k, v, ks, vs, page_table, seq_lens, batch, v_bits=4)

    def decode(self, Q: Tensor, scale: float, max_seq_len: int | None = None, out: Tensor | None = None) -> Tensor:
        """Dense GQA decode over the whole cache (``_C.fused_gqa_paged``)."""
        return _C.fused_gqa_paged(Q, self.k_pool, self.v_pool, self.k_scale, self.v_scale, self.page_table,
                                  self.seq_lens, scale, max_seq_len=max_seq_len, out=out, v_bits=self.v_bits)


RECORD_ROWS = 33  # rows of 128 bytes per (page, head): 16 of K codes, 16 of V codes, 1 of 16 + 16 fp32 scales


def fused_views(buf: Tensor, code_dtype: torch.dtype):
    """Views ``(k_pool, v_pool, k_scale, v_scale)`` over a fused page-record buffer.

    ``buf`` is uint8 ``[num_pages, Hkv, 33, 128]``: for every (page, head) the 16 K rows, the 16 V rows
    and one row holding the 16 K scales then the 16 V scales (fp32) are contiguous, so the decode kernel
    fetches a 16-token chunk with a single TMA request instead of four.  The views have the shapes every
    entry point expects (``[num_pages,Hkv,16,128]`` codes, ``[num_pages,Hkv,16]`` scales).
    """
    _C._require(buf.dtype == torch.uint8 and buf.dim() == 4 and buf.shape[2:] == (RECORD_ROWS, 128) and buf.is_contiguous(),
                "fused buffer must be contiguous uint8 [num_pages, Hkv, 33, 128]")
    k = buf[:, :, 0:16, :].view(code_dtype)
    v = buf[:, :, 16:32, :].view(code_dtype)
    sc = buf[:, :, 32, :].view(torch.float32)  # [num_pages, Hkv, 32]
    return k, v, sc[:, :, 0:16], sc[:, :, 16:32]


def pack_fused(k_pool: Tensor, v_pool: Tensor, k_scale: Tensor, v_scale: Tensor) -> Tensor:
    """Copy separate pools (page size 16, D = 128) into one fused page-record buffer."""
    num_pages, Hkv, P, D = k_pool.shape
    _C._require(P == 16 and D == 128, "fused page records need page_size 16 and head_dim 128")
    buf = torch.zeros((num_pages, Hkv, RECORD_ROWS, 128), dtype=torch.uint8, device=k_pool.device)
    k, v, ks, vs = fused_views(buf, k_pool.dtype)
    k.copy_(k_pool); v.copy_(v_pool); ks.copy_(k_scale); vs.copy_(v_scale)
    return buf


MIXED_RECORD_ROWS = 25  # 16 rows of K codes, 8 rows of 4-bit V codes (two tokens per row), 1 row of 16 + 16 fp32 scales


def mixed_views(buf: Tensor, code_dtype: torch.dtype):
    """Views ``(k_pool, v4_pool, k_scale, v_scale)`` over a buffer of mixed-precision page records.

    ``buf`` is uint8 ``[num_pages, Hkv, 25, 128]``.  K keeps 8-bit codes (``[num_pages,Hkv,16,128]`` of ``code_dtype``);
    V is stored in 4 bits, ``[num_pages,Hkv,16,64]`` uint8 with channel ``2j`` in the low and ``2j+1`` in the high
    nibble of byte ``j`` (nibble = code + 8, code in -7..7, scale = amax / 7): 200 bytes per token and head instead of
    264.  The decode kernel fetches a record with one TMA request and unpacks V in registers.
    """
    _C._require(buf.dtype == torch.uint8 and buf.dim() == 4 and buf.shape[2:] == (MIXED_RECORD_ROWS, 128) and buf.is_contiguous(),
                "mixed-precision buffer must be contiguous uint8 [num_pages, Hkv, 25, 128]")
    num_pages, Hkv = buf.shape[:2]
    k = buf[:, :, 0:16, :].view(code_dtype)
    v = buf[:, :, 16:24, :].unflatten(-1, (2, 64)).flatten(2, 3)   # [num_pages, Hkv, 16, 64]: token t = row t // 2, half t % 2
    sc = buf[:, :, 24, :].view(torch.float32)
    return k, v, sc[:, :, 0:16], sc[:, :, 16:32]


def pack_mixed(k_pool: Tensor, v4_pool: Tensor, k_scale: Tensor, v_scale: Tensor) -> Tensor:
    """Copy 8-bit K codes ``[num_pages,Hkv,16,128]``, packed 4-bit V codes ``[num_pages,Hkv,16,64]`` uint8 and their
    scales into one buffer of mixed-precision page records."""
    num_pages, Hkv, P, D = k_pool.shape
    _C._require(P == 16 and D == 128 and v4_pool.shape == (num_pages, Hkv, 16, 64) and v4_pool.dtype == torch.uint8,
                "mixed-precision records need page_size 16, head_dim 128 and uint8 [num_pages,Hkv,16,64] V codes")
    buf = torch.zeros((num_pages, Hkv, MIXED_RECORD_ROWS, 128), dtype=torch.uint8, device=k_pool.device)
    k, v, ks, vs = mixed_views(buf, k_pool.dtype)
    k.copy_(k_pool); v.copy_(v4_pool); ks.copy_(k_scale); vs.copy_(v_scale)
    return buf


def _pool_args(kv: PagedKV):
    if kv.v_bits == 4:
        kp, ks = kv.k_pool, kv.k_scale
        _C._require(kp.is_cuda and kp.dim() == 4 and kp.shape[2:] == (16, 128) and kv.v_pool.shape == (*kp.shape[:2], 16, 64)
                    and kv.v_pool.dtype == torch.uint8 and kv.v_pool.data_ptr() == kp.data_ptr() + 2048
                    and kp.stride() == (kp.shape[1] * 3200, 3200, 128, 1), "not a cache of mixed-precision page records")
        return (kp.stride(0), kp.stride(1), kp.stride(2), ks.stride(0), ks.stride(1))
    kp, ks = kv.k_pool, kv.k_scale
    _C._require(kp.is_cuda and kp.dim() == 4 and kp.stride(-1) == 1 and kv.v_pool.shape == kp.shape
                and kv.v_pool.stride() == kp.stride(), "pools must be CUDA [num_pages,Hkv,page_size,D] with one layout")
    _C._require(ks.dtype == torch.float32 and ks.shape == kp.shape[:3] and ks.stride(-1) == 1
                and kv.v_scale.stride() == ks.stride(), "scale pools must be fp32 [num_pages,Hkv,page_size]")
    return (kp.stride(0), kp.stride(1), kp.stride(2), ks.stride(0), ks.stride(1))


def build_block_meta(kv: PagedKV, block_size: int = 64, max_seq_len: int | None = None, *,
                     status: Tensor | None = None) -> Tensor:
    """Channel-wise min/max of the dequantised keys per block: fp16 ``[B, Hkv, nb, 2, D]``.

    ``status`` (optional int32 device tensor of one element) receives ``SKV_DEV_BAD_PAGE`` (2) when a page-table
    entry lies outside the pool; page 0 is read in its place."""
    strides = _pool_args(kv)
    lib = _lib.load()
    _, Hkv, P, D = kv.k_pool.shape
    N = int(max_seq_len) if max_seq_len is not None else kv.capacity
    nb = lib.skv_quest_num_blocks(N, block_size)
    meta = torch.empty((kv.batch, Hkv, nb, 2, D), dtype=torch.float16, device=kv.k_pool.device)
    dev = _C._dev_index(kv.k_pool)
    rc = lib.skv_quest_build_meta(
        kv.k_pool.data_ptr(), kv.k_scale.data_ptr(), None if kv.page_table is None else kv.page_table.data_ptr(),
        None if kv.seq_lens is None else kv.seq_lens.data_ptr(), meta.data_ptr(), kv.batch, N, Hkv, D,
        _C._code_dtype(kv.k_pool), int(block_size), P, kv.max_pages, kv.k_pool.shape[0], *strides,
        None if status is None else status.data_ptr(), dev, torch.cuda.current_stream(kv.k_pool.device).cuda_stream)
    _lib.check(rc, "build_block_meta")
    return meta


def quest_sparse_decode(Q: Tensor, kv: PagedKV, meta: Tensor, scale: float, block_size: int = 64,
                        top_k_blocks: int = 8, max_seq_len: int | None = None, return_indices: bool = False):
    """Top-k block-sparse decode with the min/max upper-bound score, exact attention inside the chosen blocks.

    Q ``[B,Hq,D]`` fp16 -> ``[B,Hq,D]`` fp16 (and the chosen block ids ``[B,Hq,top_k_blocks]`` int32).
    """
    strides = _pool_args(kv)
    _C._require(Q.is_cuda and Q.dtype == torch.float16 and Q.dim() == 3 and Q.is_contiguous(),
                "Q must be a contiguous fp16 CUDA tensor [B,Hq,D]")
    B, Hq, D = Q.shape
    _, Hkv, P, _ = kv.k_pool.shape
    _C._require(B == kv.batch, "batch mismatch between Q and the cache")
    lib = _lib.load()
    N = int(max_seq_len) if max_seq_len is not None else kv.capacity
    nb = lib.skv_quest_num_blocks(N, block_size)
    _C._require(meta.dtype == torch.float16 and meta.shape == (B, Hkv, nb, 2, D) and meta.is_contiguous(),
                "meta must be fp16 [B,Hkv,nb,2,D] built with the same block_size and max_seq_len")
    out = torch.empty((B, Hq, D), dtype=torch.float16, device=Q.device)
    idx = torch.empty((B, Hq, top_k_blocks), dtype=torch.int32, device=Q.device) if return_indices else None
    ws = _workspace.get("quest", lib.skv_quest_workspace_bytes(B, Hq, N, block_size), Q.device)
    dev = _C._dev_index(Q)
    rc = lib.skv_quest_decode(
        Q.data_ptr(), kv.k_pool.data_ptr(), kv.v_pool.data_ptr(), kv.k_scale.data_ptr(), kv.v_scale.data_ptr(),
        None if kv.page_table is None else kv.page_table.data_ptr(),
        None if kv.seq_lens is None else kv.seq_lens.data_ptr(), meta.data_ptr(), out.data_ptr(),
        None if idx is None else idx.data_ptr(), ws.data_ptr(), ws.numel(), B, N, Hq, Hkv, D,
        _C._code_dtype(kv.k_pool) | (_C.SKV_V_INT4 if kv.v_bits == 4 else 0), int(block_size), int(top_k_blocks), P,
        kv.max_pages, kv.k_pool.shape[0], *strides,
        float(scale), dev,
        torch.cuda.current_stream(Q.device).cuda_stream)
    _lib.check(rc, "quest_sparse_decode")
    return (out, idx) if return_indices else out


def rope_quant_append(qkv: Tensor, kv: PagedKV, Hq: int, rope_theta: float, *, meta: Tensor | None = None,
                      block_size: int = 64, status: Tensor | None = None) -> Tensor:
    """RoPE the new token's q and k, quantise k and v and store them at position ``seq_lens[b]`` of the cache.

    ``qkv`` ``[B, (Hq + 2*Hkv) * 128]`` fp16 or bf16 (fused projection output); returns the rotated query
    ``[B, Hq, 128]`` fp16.  ``kv.seq_lens`` is read, not advanced.  With ``meta`` (the tensor
    ``build_block_meta`` returns) the min/max metadata of the block that receives the token is updated in the
    same launch (``skv_rope_quant_append``).  A page-table entry outside the pool stores nothing and sets bit
    ``SKV_DEV_BAD_PAGE`` (2) in ``status`` (an int32 device tensor of one element), when one is given.
    """
    strides = _pool_args(kv)
    _, Hkv, P, D = kv.k_pool.shape
    B = qkv.shape[0]
    _C._require(qkv.is_cuda and qkv.dim() == 2 and qkv.is_contiguous() and qkv.shape[1] == (Hq + 2 * Hkv) * D
                and qkv.dtype in (torch.float16, torch.bfloat16), "qkv must be contiguous fp16/bf16 [B,(Hq+2Hkv)*D]")
    _C._require(kv.seq_lens is not None and B == kv.batch, "the cache needs seq_lens and a matching batch")
    if meta is not None:
        _C._require(meta.dtype == torch.float16 and meta.dim() == 5 and meta.shape[:2] == (B, Hkv) and meta.shape[3:] == (2, D)
                    and meta.is_contiguous() and meta.device == qkv.device, "meta must be fp16 [B,Hkv,nb,2,D] on qkv's device")
    q = torch.empty((B, Hq, D), dtype=torch.float16, device=qkv.device)
    rc = _lib.load().skv_rope_quant_append(
        qkv.data_ptr(), int(qkv.dtype == torch.bfloat16), q.data_ptr(), kv.k_pool.data_ptr(), kv.v_pool.data_ptr(),
        kv.k_scale.data_ptr(), kv.v_scale.data_ptr(), None if kv.page_table is None else kv.page_table.data_ptr(),
        kv.seq_lens.data_ptr(), B, Hq, Hkv, D, _C._code_dtype(kv.k_pool) | (_C.SKV_V_INT4 if kv.v_bits == 4 else 0),
        P, kv.max_pages, *strides, float(rope_theta),
        None if meta is None else meta.data_ptr(), int(block_size), 0 if meta is None else meta.shape[2],
        kv.k_pool.shape[0], None if status is None else status.data_ptr(),
        _C._dev_index(qkv), torch.cuda.current_stream(qkv.device).cuda_stream)
    _lib.check(rc, "rope_quant_append")
    return q


def repage_evicted(res, *, pool: Tensor | None = None, page_ids: Tensor | None = None) -> PagedKV:
    """Put the compacted, quantised output of ``fused_kv_evict`` back into paged form (page reclamation).

    ``res`` is the ``EvictionResult`` of a scaled-quantisation eviction in position order: codes
    ``[B, H, keep, 128]`` (int8 or e4m3) and fp32 scales ``[B, H, keep]``.  Slot ``j`` of every head's new
    sequence is that head's ``j``-th kept token (heads keep different positions; the keys already carry their
    rotary phase, so attention does not need the original positions).  The rows are written as fused page
    records of 16 tokens, either into fresh storage or -- with ``pool`` (a fused page-record buffer) and
    ``page_ids`` (int ``[B, ceil(keep/16)]``, the pages handed out by the caller's allocator) -- into an
    existing pool; the pages the sequences occupied before are then free for reuse.  Returns the ``PagedKV``
    with ``seq_lens = keep``.
    """
    K, V, ks, vs = res.K, res.V, res.k_scale, res.v_scale
    _C._require(ks is not None and vs is not None, "repage_evicted needs a scaled (int8 or fp8) eviction result")
    B, H, keep, D = K.shape
    _C._require(D == 128, "page records hold 128-channel rows")
    n = (keep + 15) // 16
    pad = n * 16 - keep

    def rows(t):      # [B,H,keep,...] -> [B*n, H, 16, ...]
        if pad:
            t = torch.cat([t, t.new_zeros((B, H, pad) + tuple(t.shape[3:]))], dim=2)
        t = t.reshape((B, H, n, 16) + tuple(t.shape[3:]))
        return t.permute(0, 2, 1, 3, *range(4, t.dim())).reshape((B * n, H, 16) + tuple(t.shape[4:]))

    code_dtype = K.dtype
    records = pack_fused(rows(K.view(torch.uint8)).view(code_dtype), rows(V.view(torch.uint8)).view(code_dtype),
                         rows(ks), rows(vs))
    if pool is None:
        table = torch.arange(B * n, dtype=torch.int32, device=K.device).view(B, n)
        buf = records
    else:
        _C._require(page_ids is not None and tuple(page_ids.shape) == (B, n), "page_ids must be [B, ceil(keep/16)]")
        _C._require(pool.dtype == torch.uint8 and pool.dim() == 4 and tuple(pool.shape[1:]) == (H, RECORD_ROWS, 128),
                    "pool must be a fused page-record buffer [num_pages, H, 33, 128]")
        pool[page_ids.reshape(-1).long()] = records
        table = page_ids.to(torch.int32).contiguous()
        buf = pool
    lens = torch.full((B,), keep, dtype=torch.int32, device=K.device)
    return PagedKV.from_fused(buf, code_dtype, table, lens, B)
