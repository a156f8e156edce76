"""Drop-in for the reference's ``sparse_kv._C`` extension module.

Same function names, argument order, tensor layouts and error type
(``RuntimeError``) as the pybind module defined in the reference's
``csrc/pybind/bindings.cpp:19-31``; the work is done by the sm_100a kernels
behind the C-ABI of ``include/skv_b200.h``.  Arguments the reference does not
have are keyword-only, so every reference call site runs unchanged.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _lib, _workspace


def _dev_index(t: Tensor) -> int:
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _kv_strides(K: Tensor, V: Tensor, what: str) -> tuple[int, int, int]:
    _require(K.stride(-1) == 1 and V.stride(-1) == 1, f"{what}: the channel dimension of K/V must be contiguous")
    _require(K.stride() == V.stride(), f"{what}: K and V must share one memory layout")
    return K.stride(0), K.stride(1), K.stride(2)


def fused_gqa(Q: Tensor, K: Tensor, V: Tensor, scale: float, *, seq_lens: Tensor | None = None,
              out: Tensor | None = None, mass: Tensor | None = None) -> Tensor:
    """Dense GQA decode attention; reference: ``launch_fused_gqa`` (csrc/kernels/gqa_decode.cu:218-290).

    Q ``[B, Hq, D]`` fp16, K/V ``[B, N, Hkv, D]`` fp16, returns ``[B, Hq, D]`` fp16 with
    ``Out[b,h] = softmax(scale * Q[b,h] K[b,:,h // (Hq/Hkv)]^T) V[b,:,h // (Hq/Hkv)]``.
    Unlike the reference, K/V may be any strided view with a contiguous channel
    dimension (for example ``cache.permute(0, 2, 1, 3)`` of a ``[B, Hkv, N, D]``
    cache), D may be 64 or 128, the launch goes to the current stream of Q's
    device, and ``seq_lens`` (int32 ``[B]``) bounds the tokens read per sequence.
    ``mass`` (fp32 ``[B, Hkv, N]``, optional) receives, added in place, every token's attention probability
    summed over the query heads of its kv-head: the running ``scores`` of ``fused_kv_evict``.
    """
    _require(Q.is_cuda and K.is_cuda and V.is_cuda, "Q/K/V must be CUDA tensors")
    _require(Q.dtype == torch.float16 and K.dtype == torch.float16 and V.dtype == torch.float16,
             "all inputs must be fp16")
    _require(Q.dim() == 3 and K.dim() == 4 and V.dim() == 4, "expected Q [B,Hq,D] and K/V [B,N,Hkv,D]")
    _require(Q.is_contiguous(), "Q must be contiguous")
    B, Hq, D = Q.shape
    N, Hkv = K.shape[1], K.shape[2]
    _require(K.shape[0] == B and V.shape[0] == B, "batch size mismatch across Q/K/V")
    _require(K.shape[3] == D and V.shape[3] == D, f"K/V head_dim must match Q head_dim={D}")
    _require(V.shape[1] == N and V.shape[2] == Hkv, "V shape must be [B, N, Hkv, D] matching K")
    _require(Hkv > 0 and Hq % Hkv == 0, f"Hq={Hq} must be divisible by Hkv={Hkv}")
    _require(K.device == Q.device and V.device == Q.device, "Q/K/V must be on one device")
    sb, sn, sh = _kv_strides(K, V, "fused_gqa")
    dev = _dev_index(Q)
    lib = _lib.load()
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.float16, device=Q.device)
    else:
        _require(out.shape == (B, Hq, D) and out.dtype == torch.float16 and out.is_contiguous()
                 and out.device == Q.device, "out must be a contiguous fp16 [B,Hq,D] tensor on Q's device")
    lens_ptr = None
    if seq_lens is not None:
        _require(seq_lens.dtype == torch.int32 and seq_lens.shape == (B,) and seq_lens.device == Q.device
                 and seq_lens.is_contiguous(), "seq_lens must be a contiguous int32 [B] tensor on Q's device")
        lens_ptr = seq_lens.data_ptr()
    stream = torch.cuda.current_stream(Q.device).cuda_stream
    if mass is not None:
        _require(mass.dtype == torch.float32 and mass.shape == (B, Hkv, N) and mass.is_contiguous()
                 and mass.device == Q.device, "mass must be a contiguous fp32 [B,Hkv,N] tensor on Q's device")
        ws = _workspace.get("gqa_mass", lib.skv_gqa_decode_mass_workspace_bytes(B, N, Hq, Hkv, D, dev), Q.device)
        rc = lib.skv_gqa_decode_mass(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), mass.data_ptr(),
                                     ws.data_ptr(), ws.numel(), B, N, Hq, Hkv, D, sb, sn, sh, lens_ptr, float(scale),
                                     dev, stream)
        _lib.check(rc, "fused_gqa")
        return out
    nbytes = lib.skv_gqa_decode_workspace_bytes(B, N, Hq, Hkv, D, dev)
    ws = _workspace.get("gqa", nbytes, Q.device)
    rc = lib.skv_gqa_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                            B, N, Hq, Hkv, D, _lib.KV_F16, None, None, sb, sn, sh, lens_ptr, float(scale), dev, stream)
    _lib.check(rc, "fused_gqa")
    return out


def token_sparse_decode(Q: Tensor, K: Tensor, V: Tensor, top_k: int, sink_tokens: int = 0, *,
                        return_indices: bool = False):
    """Token-level top-k sparse attention on fp16 CUDA tensors.

    Q ``[B,H,S,D]``, K/V ``[B,H,T,D]`` -> ``[B,H,S,D]`` fp16: softmax over the ``top_k`` best keys and the
    first ``sink_tokens`` positions only (sparse_kv/attention.py:25-38).  With ``return_indices`` also
    returns the selected key positions ``[B,H,S,top_k]`` int32, ascending, -1 padded.
    """
    _require(Q.is_cuda and K.is_cuda and V.is_cuda, "Q/K/V must be CUDA tensors")
    _require(Q.dtype == torch.float16, "Q must be fp16")
    _require(K.dtype == torch.float16, "K must be fp16")
    _require(V.dtype == torch.float16, "V must be fp16")
    _require(Q.dim() == 4 and K.dim() == 4 and V.dim() == 4, "expected Q [B,H,S,D] and K/V [B,H,T,D]")
    B, H, S, D = Q.shape
    T = K.shape[2]
    _require(K.shape[0] == B and K.shape[1] == H, "K batch/head dims must match Q")
    _require(K.shape[3] == D and V.shape == K.shape, "V shape must match K")
    _require(top_k > 0, "top_k must be positive")
    _require(K.device == Q.device and V.device == Q.device, "Q/K/V must be on one device")
    if Q.stride(-1) != 1:
        Q = Q.contiguous()
    sb, sh, st = _kv_strides(K, V, "token_sparse_decode")
    dev = _dev_index(Q)
    lib = _lib.load()
    out = torch.empty((B, H, S, D), dtype=torch.float16, device=Q.device)
    idx = torch.empty((B, H, S, top_k), dtype=torch.int32, device=Q.device) if return_indices else None
    ws = _workspace.get("token_sparse", lib.skv_token_sparse_workspace_bytes(B, H, S, T), Q.device)
    stream = torch.cuda.current_stream(Q.device).cuda_stream
    rc = lib.skv_token_sparse_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(),
                                     None if idx is None else idx.data_ptr(), ws.data_ptr(), ws.numel(),
                                     B, H, S, T, D, Q.stride(0), Q.stride(1), Q.stride(2), sb, sh, st,
                                     int(top_k), int(sink_tokens), float(D) ** -0.5, dev, stream)
    _lib.check(rc, "token_sparse_decode")
    return (out, idx) if return_indices else out


def kv_evict_quant_forward(Q: Tensor, K: Tensor, V: Tensor, top_k: int, use_int8: bool) -> Tensor:
    """Reference binding ``kv_evict_quant_forward(Q, K, V, top_k, use_int8)`` (csrc/kernels/kv_evict_quant.cu:272-364).

    Despite its name it is token-sparse attention: Q ``[B,H,1,D]``, K/V ``[B,H,T,D]`` fp16 -> ``[B,H,1,D]``.
    As in the reference, ``use_int8=True`` is rejected (kv_evict_quant.cu:294).  The top-k here is exact.
    """
    _require(not use_int8, "INT8 path not enabled in this build")
    return token_sparse_decode(Q, K, V, top_k, 0)


def sparse_attention_forward(Q: Tensor, K: Tensor, V: Tensor, block_size: int, top_k_blocks: int, *,
                             return_indices: bool = False):
    """Reference binding ``sparse_attention_forward`` (csrc/kernels/sparse_attention.cu:178-244).

    Q ``[B,H,1,D]``, K/V ``[B,H,T,D]`` fp16 -> ``[B,H,1,D]`` fp16: blocks of ``block_size`` tokens are scored by
    the mean of ``q.k / sqrt(D)``, the ``top_k_blocks`` best are soft-maxed on those scores and the output is
    the weighted sum of their mean value vectors.  ``return_indices`` also returns the chosen block ids
    ``[B,H,top_k_blocks]`` int32 (ascending, -1 padded), which the reference computes but drops.
    """
    _require(Q.is_cuda and K.is_cuda and V.is_cuda, "Q/K/V must be CUDA")
    _require(Q.dtype == torch.float16, "Q must be fp16")
    _require(K.dtype == torch.float16, "K must be fp16")
    _require(V.dtype == torch.float16, "V must be fp16")
    _require(Q.dim() == 4 and K.dim() == 4 and V.dim() == 4, "expected Q [B,H,1,D] and K/V [B,H,T,D]")
    _require(Q.shape[2] == 1, "sparse_attention_forward: Q must be decode-step shape [B,H,1,D]")
    _require(K.shape[0] == Q.shape[0] and K.shape[1] == Q.shape[1], "K batch/head dims must match Q")
    _require(V.shape[2] == K.shape[2] and V.shape[3] == K.shape[3] and K.shape[3] == Q.shape[3], "V shape must match K")
    _require(top_k_blocks > 0, "top_k_blocks must be positive")
    _require(block_size > 0, "block_size must be positive")
    B, H, _, D = Q.shape
    T = K.shape[2]
    if Q.stride(-1) != 1:
        Q = Q.contiguous()
    sb, sh, st = _kv_strides(K, V, "sparse_attention_forward")
    dev = _dev_index(Q)
    lib = _lib.load()
    out = torch.empty((B, H, 1, D), dtype=torch.float16, device=Q.device)
    idx = torch.empty((B, H, top_k_blocks), dtype=torch.int32, device=Q.device) if return_indices else None
    ws = _workspace.get("block_sparse", lib.skv_block_sparse_workspace_bytes(B, H, T, block_size), Q.device)
    stream = torch.cuda.current_stream(Q.device).cuda_stream
    rc = lib.skv_block_sparse_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(),
                                     None if idx is None else idx.data_ptr(), ws.data_ptr(), ws.numel(),
                                     B, H, T, D, Q.stride(0), Q.stride(1), sb, sh, st, int(block_size),
                                     int(top_k_blocks), float(D) ** -0.5, dev, stream)
    _lib.check(rc, "sparse_attention_forward")
    return (out, idx) if return_indices else out


SKV_OUT_BF16 = 0x100  # OR-ed into the kv_dtype argument of skv_gqa_decode_paged: bf16 output elements
SKV_V_INT4 = 0x200    # ... and of skv_rope_quant_append: V is 4-bit (mixed-precision page records)
SKV_EARLY_EXCEPT_LAST = 0x400   # skv_gqa_decode_paged: the previous kernel wrote only the query and each sequence's last token


def _code_dtype(t: Tensor) -> int:
    if t.dtype == torch.int8:
        return _lib.KV_I8
    if t.dtype == torch.float8_e4m3fn:
        return _lib.KV_E4M3
    raise RuntimeError("8-bit KV pools must be int8 or float8_e4m3fn")


def fused_gqa_paged(Q: Tensor, k_pool: Tensor, v_pool: Tensor, k_scale: Tensor, v_scale: Tensor,
                    page_table: Tensor | None, seq_lens: Tensor | None, scale: float, *,
                    max_seq_len: int | None = None, out: Tensor | None = None, v_bits: int = 8,
                    after_append: bool = False) -> Tensor:
    """Dense GQA decode over a paged INT8 / FP8-E4M3 cache with per-token-per-head fp32 scales.

    ``after_append=True``: the kernel launched just before this call on the same stream was ``paged.rope_quant_append``
    for the same step (it wrote the query and each sequence's last token, nothing else this call reads, and
    ``seq_lens`` / ``page_table`` are older than it): the decode kernel then streams the rest of the cache while that
    kernel is still running (``SKV_EARLY_EXCEPT_LAST``).
    ``v_bits=4``: the pools are the views of a mixed-precision record buffer (``paged.mixed_views``): ``v_pool`` is
    uint8 ``[num_pages, Hkv, 16, 64]`` of packed 4-bit codes, ``k_pool`` stays 8-bit.

    Q ``[B,Hq,128]`` fp16; pools ``[num_pages, Hkv, page_size, 128]`` int8 or float8_e4m3fn; scale pools
    ``[num_pages, Hkv, page_size]`` fp32; ``page_table`` int32 ``[B, max_pages]`` (``None``: sequence b owns
    pages ``b*max_pages ...``, so a ``[B,Hkv,T,128]`` compacted cache is passed with ``page_size = T``);
    ``seq_lens`` int32 ``[B]``.  Returns ``[B,Hq,128]`` fp16, or bf16 when ``out`` is a bf16 tensor.  No
    reference counterpart.
    """
    _require(Q.is_cuda and Q.dtype == torch.float16 and Q.dim() == 3 and Q.is_contiguous(),
             "Q must be a contiguous fp16 CUDA tensor [B,Hq,D]")
    _require(v_bits in (4, 8), "v_bits must be 4 or 8")
    kvt = _code_dtype(k_pool)
    B, Hq, D = Q.shape
    _require(k_pool.dim() == 4, "k_pool must be [num_pages,Hkv,page_size,D]")
    num_pages, Hkv, P, Dk = k_pool.shape
    _require(Dk == D, "pool head_dim must match Q")
    if v_bits == 4:
        _require(v_pool.dtype == torch.uint8 and v_pool.shape == (num_pages, Hkv, P, D // 2) and k_pool.stride(-1) == 1,
                 "with v_bits=4, v_pool must be uint8 [num_pages,Hkv,page_size,D/2] of packed 4-bit codes")
        kvt |= SKV_V_INT4
    else:
        _require(v_pool.shape == k_pool.shape and k_pool.dtype == v_pool.dtype,
                 "k_pool and v_pool must both be [num_pages,Hkv,page_size,D] of one 8-bit dtype")
        _require(k_pool.stride(-1) == 1 and k_pool.stride() == v_pool.stride(), "pools must share a channel-contiguous layout")
    _require(k_scale.shape == (num_pages, Hkv, P) and v_scale.shape == k_scale.shape and k_scale.dtype == torch.float32
             and v_scale.dtype == torch.float32 and k_scale.stride() == v_scale.stride() and k_scale.stride(-1) == 1,
             "scale pools must be fp32 [num_pages,Hkv,page_size] with one layout")
    if page_table is not None:
        _require(page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.shape[0] == B
                 and page_table.is_contiguous() and page_table.device == Q.device, "page_table must be int32 [B,max_pages]")
        max_pages = page_table.shape[1]
    else:
        _require(num_pages % B == 0, "without a page table num_pages must be B * max_pages")
        max_pages = num_pages // B
    if seq_lens is not None:
        _require(seq_lens.dtype == torch.int32 and seq_lens.shape == (B,) and seq_lens.is_contiguous()
                 and seq_lens.device == Q.device, "seq_lens must be a contiguous int32 [B] tensor on Q's device")
    N = int(max_seq_len) if max_seq_len is not None else max_pages * P
    _require(0 < N <= max_pages * P, "max_seq_len must be in (0, max_pages * page_size]")
    dev = _dev_index(Q)
    lib = _lib.load()
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.float16, device=Q.device)
    _require(out.dtype in (torch.float16, torch.bfloat16) and out.shape == (B, Hq, D) and out.is_contiguous()
             and out.device == Q.device, "out must be a contiguous fp16 or bf16 [B,Hq,D] tensor on Q's device")
    if out.dtype == torch.bfloat16:
        kvt |= SKV_OUT_BF16
    if after_append:
        kvt |= SKV_EARLY_EXCEPT_LAST
    ws = _workspace.get("gqa", lib.skv_gqa_decode_workspace_bytes(B, N, Hq, Hkv, D, dev), Q.device)
    stream = torch.cuda.current_stream(Q.device).cuda_stream
    rc = lib.skv_gqa_decode_paged(
        Q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(),
        None if page_table is None else page_table.data_ptr(), None if seq_lens is None else seq_lens.data_ptr(),
        out.data_ptr(), ws.data_ptr(), ws.numel(), B, N, Hq, Hkv, D, kvt, P, max_pages, num_pages,
        k_pool.stride(0), k_pool.stride(1), k_pool.stride(2), k_scale.stride(0), k_scale.stride(1),
        float(scale), dev, stream)
    _lib.check(rc, "fused_gqa_paged")
    return out
