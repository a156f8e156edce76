"""Mixed-precision page records (8-bit K, 4-bit V): decode against the oracle on the dequantised cache, and the
append kernel's 4-bit quantiser against the oracle's rule, bit for bit."""
import pytest
import torch

from llm_inference_optimization_b200 import _C, _workspace, paged
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3
D = 128


def make_case(B, Hq, Hkv, T, fmt, seed, unit=False):
    g = torch.Generator().manual_seed(seed)
    s = 1.0 if unit else D ** -0.5
    Q = (torch.randn(B, Hq, D, generator=g) * s).half()
    K = (torch.randn(B, Hkv, T, D, generator=g) * s).half()
    V = (torch.randn(B, Hkv, T, D, generator=g) * s).half()
    kc, ks = (oracle.quantize_e4m3 if fmt == "fp8" else oracle.quantize_int8)(K)
    vc, vs = oracle.quantize_int4(V)
    perm = torch.randperm(B * (T // 16) + 5, generator=g)
    kp, ksp, table = oracle.build_paged_cache(kc, ks, 16, perm)
    vp, vsp, _ = oracle.build_paged_cache(vc, vs, 16, perm)
    Kd, Vd = oracle.dequantize(kc, ks), oracle.dequantize_int4(vc, vs)
    return Q, V, (kp, vp, ksp, vsp, table), (Kd.permute(0, 2, 1, 3), Vd.permute(0, 2, 1, 3))


def mixed_cache(pools, dev, lens, B):
    kp, vp, ksp, vsp, table = (t.to(dev) for t in pools)
    buf = paged.pack_mixed(kp, vp, ksp, vsp)
    sl = None if lens is None else torch.tensor(lens, dtype=torch.int32, device=dev)
    return paged.PagedKV.from_mixed(buf, kp.dtype, table, sl, B)


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
@pytest.mark.parametrize("B,Hq,Hkv,T,lens", [(1, 32, 8, 4096, None), (3, 32, 8, 2048, [2048, 1, 1037]),
                                             (2, 8, 2, 8192, [8192, 5000]), (1, 8, 1, 64, [17]),
                                             (1, 4, 4, 1024, [1000]), (1, 12, 2, 1024, None), (2, 16, 2, 4096, [0, 4096])])
def test_decode_matches_oracle_on_dequantised_cache(cuda_device, fmt, B, Hq, Hkv, T, lens):
    Q, _, pools, (Kd, Vd) = make_case(B, Hq, Hkv, T, fmt, seed=T + B)
    kv = mixed_cache(pools, cuda_device, lens, B)
    scale = D ** -0.5
    out = kv.decode(Q.to(cuda_device), scale)
    torch.cuda.synchronize()
    assert _workspace.status(_workspace.get("gqa", 0, cuda_device)) == 0
    want = oracle.dense_gqa_decode(Q, Kd, Vd, scale, None if lens is None else torch.tensor(lens, dtype=torch.int32))
    assert (out.float().cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
def test_unit_variance_long_context_and_bf16_output(cuda_device, fmt):
    """N(0,1) values at 32K tokens for 16 sequences' worth of CTAs per SM slot: the bias of the 4-bit codes (1032 per
    element) is taken out of fp32 accumulators that have summed thousands of tokens."""
    Q, V, pools, (Kd, Vd) = make_case(2, 32, 8, 32768, fmt, seed=3, unit=True)
    kv = mixed_cache(pools, cuda_device, None, 2)
    scale = D ** -0.5
    out = torch.empty(2, 32, D, dtype=torch.bfloat16, device=cuda_device)
    kv.decode(Q.to(cuda_device), scale, out=out)
    want = oracle.dense_gqa_decode(Q, Kd, Vd, scale)
    assert (out.float().cpu() - want).abs().max().item() <= 2.0 ** -8 * max(1.0, want.abs().max().item()) + TOL
    # what 4 bits cost against the unquantised V: the error of a softmax-weighted mean of per-token roundings
    exact = oracle.dense_gqa_decode(Q, Kd, V.float().permute(0, 2, 1, 3), scale)
    rel = (want - exact).norm() / exact.norm()
    print(f"4-bit V against fp16 V ({fmt} K): relative output error {rel:.4f}")
    assert rel < 0.15


def test_more_than_eight_heads_per_group_is_refused(cuda_device):
    Q, _, pools, _ = make_case(1, 32, 2, 256, "int8", seed=1)
    kv = mixed_cache(pools, cuda_device, None, 1)
    with pytest.raises(RuntimeError):
        kv.decode(Q.to(cuda_device), D ** -0.5)


@pytest.mark.parametrize("dtype,code_dtype", [(torch.bfloat16, torch.float8_e4m3fn), (torch.float16, torch.int8)])
def test_append_quantises_v_to_four_bits_like_the_oracle(cuda_device, dtype, code_dtype):
    B, Hq, Hkv, pages_per_seq = 3, 8, 2, 4
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    qkv[1, (Hq + Hkv) * D:(Hq + Hkv + 1) * D] = 0          # an all-zero V row: scale 1.0, codes 8
    buf = torch.zeros(B * pages_per_seq + 2, Hkv, paged.MIXED_RECORD_ROWS, 128, dtype=torch.uint8, device=cuda_device)
    table = torch.randperm(B * pages_per_seq + 2, generator=g)[:B * pages_per_seq].view(B, pages_per_seq).to(torch.int32).to(cuda_device)
    lens = torch.tensor([0, 17, 63], dtype=torch.int32, device=cuda_device)
    kv = paged.PagedKV.from_mixed(buf, code_dtype, table, lens, B)
    q = paged.rope_quant_append(qkv.to(cuda_device), kv, Hq, 500000.0)
    torch.cuda.synchronize()
    assert torch.isfinite(q.float()).all()
    v = qkv.float().view(B, Hq + 2 * Hkv, D)[:, Hq + Hkv:]            # [B, Hkv, D], the rounded inputs themselves
    codes, scales = oracle.quantize_int4(v)
    for b in range(B):
        pos = int(lens[b])
        page, slot = int(table[b, pos // 16]), pos % 16
        assert torch.equal(kv.v_pool[page, :, slot].cpu(), codes[b])
        assert torch.equal(kv.v_scale[page, :, slot].cpu(), scales[b])
    assert torch.equal(kv.v_pool[int(table[1, 1]), 0, 1].cpu(), torch.full((64,), 0x88, dtype=torch.uint8))
    # nothing but the three (page, slot) rows was written to the V area
    assert int((kv.v_pool != 0).any(dim=-1).sum()) == B * Hkv
    # the step's attention over the cache with the new token in place agrees with the oracle
    new_lens = (lens + 1).cpu()
    kv2 = paged.PagedKV.from_mixed(buf, code_dtype, table, (lens + 1), B)
    out = kv2.decode(q, D ** -0.5)
    T = pages_per_seq * 16
    Kd = torch.zeros(B, T, Hkv, D)
    Vd = torch.zeros(B, T, Hkv, D)
    k8, v4, ks, vs = (t.cpu() for t in paged.mixed_views(buf, code_dtype))
    for b in range(B):
        pg = table[b].cpu().long()
        Kd[b] = oracle.dequantize(k8[pg], ks[pg]).permute(0, 2, 1, 3).reshape(T, Hkv, D)
        Vd[b] = oracle.dequantize_int4(v4[pg], vs[pg]).permute(0, 2, 1, 3).reshape(T, Hkv, D)
    want = oracle.dense_gqa_decode(q.cpu(), Kd, Vd, D ** -0.5, new_lens)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
def test_quest_block_sparse_decode_over_mixed_precision_pages(cuda_device, fmt):
    """The Quest path (metadata from the 8-bit keys, exact attention inside the chosen blocks) reads 4-bit values too."""
    from llm_inference_optimization_b200 import workloads
    B, Hq, Hkv, T = 2, 8, 2, 4096
    Q, K, V, _ = workloads.planted_block_cache(B, Hq, Hkv, T, seed=9)
    Q, K, V = Q.half(), K.half(), V.half()
    kc, ks = (oracle.quantize_e4m3 if fmt == "fp8" else oracle.quantize_int8)(K)
    vc, vs = oracle.quantize_int4(V)
    perm = torch.randperm(B * (T // 16) + 3, generator=torch.Generator().manual_seed(2))
    kp, ksp, table = oracle.build_paged_cache(kc, ks, 16, perm)
    vp, vsp, _ = oracle.build_paged_cache(vc, vs, 16, perm)
    lens = [T, 1500]
    kv = mixed_cache((kp, vp, ksp, vsp, table), cuda_device, lens, B)
    meta = paged.build_block_meta(kv, 64)
    out, idx = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, D ** -0.5, 64, 8, return_indices=True)
    torch.cuda.synchronize()
    Kd, Vd = oracle.dequantize(kc, ks), oracle.dequantize_int4(vc, vs)
    want = oracle.attend_selected_blocks(Q, Kd, Vd, idx.cpu().long(), 64, D ** -0.5, torch.tensor(lens, dtype=torch.int32))
    assert (out.float().cpu() - want).abs().max().item() <= TOL
    with pytest.raises(RuntimeError):   # more than 512 gathered tokens are not served over 4-bit values
        paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, D ** -0.5, 64, 16)
