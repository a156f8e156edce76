"""Dense decode over a paged INT8 / FP8 cache vs the oracle on the dequantised cache (max-abs <= 2e-3)."""
import pytest
import torch

from llm_inference_optimization_b200 import _C, _workspace
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def make_case(B, Hq, Hkv, T, fmt, seed, page_size=16, unit=False):
    g = torch.Generator().manual_seed(seed)
    D = 128
    s = 1.0 if unit else D ** -0.5
    Q = (torch.randn(B, Hq, D, generator=g) * s).half()
    K = (torch.randn(B, Hkv, T, D, generator=g) * s).half()
    V = (torch.randn(B, Hkv, T, D, generator=g) * s).half()
    quant = oracle.quantize_e4m3 if fmt == "fp8" else oracle.quantize_int8
    kc, ks = quant(K)
    vc, vs = quant(V)
    pps = T // page_size
    perm = torch.randperm(B * pps + 5, generator=g)  # a few unused pages in the pool
    kp, ksp, table = oracle.build_paged_cache(kc, ks, page_size, perm)
    vp, vsp, _ = oracle.build_paged_cache(vc, vs, page_size, perm)
    Kd, Vd = oracle.dequantize(kc, ks), oracle.dequantize(vc, vs)  # [B,Hkv,T,D] fp32
    return Q, (kp, vp, ksp, vsp, table), (Kd.permute(0, 2, 1, 3), Vd.permute(0, 2, 1, 3))


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
@pytest.mark.parametrize("B,Hq,Hkv,T,lens", [(1, 32, 8, 4096, None), (3, 32, 8, 2048, [2048, 1, 1037]),
                                             (2, 8, 2, 8192, [8192, 5000]), (1, 16, 1, 64, [17]),
                                             # group sizes 16 (two head tiles), 8, 1 (no grouping) and 6 (not a power of two)
                                             (2, 32, 2, 4096, [4096, 777]), (1, 16, 2, 2048, None),
                                             (1, 4, 4, 1024, [1000]), (1, 12, 2, 1024, None)])
def test_paged_decode(cuda_device, fmt, B, Hq, Hkv, T, lens):
    Q, pools, (Kd, Vd) = make_case(B, Hq, Hkv, T, fmt, seed=T + B)
    kp, vp, ksp, vsp, table = (t.to(cuda_device) for t in pools)
    sl = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    scale = 128 ** -0.5
    out = _C.fused_gqa_paged(Q.to(cuda_device), kp, vp, ksp, vsp, table, None if sl is None else sl.to(cuda_device), scale)
    torch.cuda.synchronize()
    assert _workspace.status(_workspace.get("gqa", 0, cuda_device)) == 0
    want = oracle.dense_gqa_decode(Q, Kd, Vd, scale, sl)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
def test_unit_variance_long_context(cuda_device, fmt):
    """N(0,1) values at 64K tokens: exercises scale folding and the running-max rescale."""
    Q, pools, (Kd, Vd) = make_case(1, 32, 8, 65536, fmt, seed=3, unit=True)
    kp, vp, ksp, vsp, table = (t.to(cuda_device) for t in pools)
    scale = 128 ** -0.5
    out = _C.fused_gqa_paged(Q.to(cuda_device), kp, vp, ksp, vsp, table, None, scale)
    want = oracle.dense_gqa_decode(Q, Kd, Vd, scale)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
def test_fused_page_records(cuda_device, fmt):
    """K codes, V codes and scales of a page in one 33-row record: same result, one TMA request per chunk."""
    from llm_inference_optimization_b200 import paged
    B, Hq, Hkv, T = 2, 32, 8, 8192
    Q, pools, (Kd, Vd) = make_case(B, Hq, Hkv, T, fmt, seed=77)
    kp, vp, ksp, vsp, table = (t.to(cuda_device) for t in pools)
    lens = torch.tensor([8192, 4999], dtype=torch.int32)
    buf = paged.pack_fused(kp, vp, ksp, vsp)
    kv = paged.PagedKV.from_fused(buf, kp.dtype, table, lens.to(cuda_device), B)
    assert kv.v_pool.data_ptr() == kv.k_pool.data_ptr() + 2048
    scale = 128 ** -0.5
    out = kv.decode(Q.to(cuda_device), scale)
    torch.cuda.synchronize()
    assert _workspace.status(_workspace.get("gqa", 0, cuda_device)) == 0
    want = oracle.dense_gqa_decode(Q, Kd, Vd, scale, lens)
    assert (out.float().cpu() - want).abs().max().item() <= TOL
    sep = _C.fused_gqa_paged(Q.to(cuda_device), kp, vp, ksp, vsp, table, lens.to(cuda_device), scale)
    assert (out.float() - sep.float()).abs().max().item() <= 1e-3


def test_compacted_cache_without_page_table(cuda_device):
    """The [B,H,keep,D] codes + [B,H,keep] scales an eviction produces are read as one page per sequence."""
    g = torch.Generator().manual_seed(9)
    B, Hq, Hkv, T = 2, 8, 2, 4160
    Q = torch.randn(B, Hq, 128, generator=g).half()
    K = torch.randn(B, Hkv, T, 128, generator=g).half()
    V = torch.randn(B, Hkv, T, 128, generator=g).half()
    kc, ks = oracle.quantize_int8(K)
    vc, vs = oracle.quantize_int8(V)
    out = _C.fused_gqa_paged(Q.to(cuda_device), kc.view(B, Hkv, T, 128).to(cuda_device), vc.to(cuda_device),
                             ks.to(cuda_device), vs.to(cuda_device), None, None, 128 ** -0.5)
    want = oracle.dense_gqa_decode(Q, oracle.dequantize(kc, ks).permute(0, 2, 1, 3),
                                   oracle.dequantize(vc, vs).permute(0, 2, 1, 3), 128 ** -0.5)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("B,Hq,Hkv,T,lens", [(5, 4, 1, 8192, [8192, 17, 5000, 64, 1000]), (3, 8, 2, 4096, [4096, 4096, 4096]),
                                             (4, 4, 1, 2048, [1, 2048, 0, 700]), (16, 4, 1, 1024, None)])
def test_ragged_batch_work_list_schedule(cuda_device, lib, B, Hq, Hkv, T, lens):
    """A ragged batch with few (sequence, kv-head) pairs is scheduled from a work list that every CTA derives from
    seq_lens (one wave of nearly equal CTAs) instead of the host's plan for the longest sequence: same output as that
    plan and as the oracle, with an empty sequence, a one-token sequence and equal lengths among the cases."""
    Q, pools, (Kd, Vd) = make_case(B, Hq, Hkv, T, "fp8", seed=B * T)
    kp, vp, ksp, vsp, table = (t.to(cuda_device) for t in pools)
    sl = torch.tensor(lens if lens is not None else [T - 37 * i for i in range(B)], dtype=torch.int32)
    scale = 128 ** -0.5
    outs = {}
    try:
        for mode in (1, 0):
            assert lib.skv_gqa_set_ragged_worklist(mode) == 0
            outs[mode] = _C.fused_gqa_paged(Q.to(cuda_device), kp, vp, ksp, vsp, table, sl.to(cuda_device), scale)
            torch.cuda.synchronize()
            assert _workspace.status(_workspace.get("gqa", 0, cuda_device)) == 0
    finally:
        lib.skv_gqa_set_ragged_worklist(1)
    want = oracle.dense_gqa_decode(Q, Kd, Vd, scale, sl)
    for mode in (1, 0):
        assert (outs[mode].float().cpu() - want).abs().max().item() <= TOL, mode


def test_decode_overlapping_the_append_kernel_reads_the_appended_token(cuda_device):
    """after_append=True lets the decode kernel stream the cache while the append kernel of the same step is still
    running; only the tile that holds the appended token waits.  Fifty steps of append + decode over sequences whose
    lengths cross tile and page boundaries must equal the ordered launch bit for bit."""
    from llm_inference_optimization_b200 import paged
    B, Hq, Hkv, D, pages_per_seq = 6, 8, 2, 128, 24
    g = torch.Generator().manual_seed(21)
    total = B * pages_per_seq
    buf = torch.randint(0, 256, (total, Hkv, paged.RECORD_ROWS, 128), generator=g, dtype=torch.uint8)
    buf[:, :, :32] = torch.where((buf[:, :, :32] & 0x7F) == 0x7F, buf[:, :, :32] & 0xFE, buf[:, :, :32])
    buf = buf.to(cuda_device)
    table = torch.randperm(total, generator=g).view(B, pages_per_seq).to(torch.int32).to(cuda_device)
    lens0 = torch.tensor([0, 62, 63, 64, 127, 300], dtype=torch.int32)
    outs = {}
    for overlap in (True, False):
        work = buf.clone()
        kv = paged.PagedKV.from_fused(work, torch.float8_e4m3fn, table, lens0.to(cuda_device).clone(), B)
        kv.k_scale.fill_(0.01)
        kv.v_scale.fill_(0.01)
        gs = torch.Generator().manual_seed(5)
        res = []
        for step in range(50):
            qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=gs).to(torch.bfloat16).to(cuda_device)
            q = paged.rope_quant_append(qkv, kv, Hq, 500000.0)
            new_lens = kv.seq_lens + 1
            out = _C.fused_gqa_paged(q, kv.k_pool, kv.v_pool, kv.k_scale, kv.v_scale, table, new_lens, D ** -0.5,
                                     after_append=overlap)
            kv.seq_lens.copy_(new_lens)
            res.append(out)
        torch.cuda.synchronize()
        assert _workspace.status(_workspace.get("gqa", 0, cuda_device)) == 0
        outs[overlap] = torch.stack(res)
    assert torch.isfinite(outs[True].float()).all()
    assert torch.equal(outs[True], outs[False])
