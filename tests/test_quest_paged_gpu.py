"""Quest-style block-sparse decode over a paged FP8 / INT8 cache: metadata, block sets and outputs vs the oracle."""
import pytest
import torch

from llm_inference_optimization_b200 import paged, workloads
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def paged_case(Q, K, V, fmt, dev, seed, page_size=16, seq_lens=None):
    quant = oracle.quantize_e4m3 if fmt == "fp8" else oracle.quantize_int8
    kc, ks = quant(K)
    vc, vs = quant(V)
    B, Hkv, T, D = K.shape
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(B * (T // page_size) + 3, generator=g)
    kp, ksp, table = oracle.build_paged_cache(kc, ks, page_size, perm)
    vp, vsp, _ = oracle.build_paged_cache(vc, vs, page_size, perm)
    kv = paged.PagedKV(kp.to(dev), vp.to(dev), ksp.to(dev), vsp.to(dev), table.to(dev),
                       None if seq_lens is None else seq_lens.to(dev), B)
    return kv, oracle.dequantize(kc, ks), oracle.dequantize(vc, vs)


def score_gap(scores, k):
    if k >= scores.shape[-1]:
        return 1.0
    v = scores.topk(k + 1, -1).values
    return (v[..., k - 1] - v[..., k]).min().item()


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
@pytest.mark.parametrize("B,Hq,Hkv,T,bs,k", [(2, 32, 8, 8192, 64, 8), (1, 8, 2, 1024, 64, 4), (1, 4, 4, 512, 32, 16)])
def test_meta_blocks_and_outputs(cuda_device, fmt, B, Hq, Hkv, T, bs, k):
    Q, K, V, _ = workloads.planted_block_cache(B, Hq, Hkv, T, block_size=bs, planted=min(8, T // bs))
    kv, Kd, Vd = paged_case(Q, K, V, fmt, cuda_device, seed=T)
    meta = paged.build_block_meta(kv, bs)
    want_meta = oracle.block_minmax_meta(Kd, bs)
    assert torch.equal(meta.cpu(), want_meta)                     # metadata bit-exact
    scale = 128 ** -0.5
    out, idx = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, scale, bs, k, return_indices=True)
    sc = oracle.quest_block_scores(Q, want_meta, scale)
    blocks = oracle.topk_blocks(sc, k)
    if score_gap(sc, k) > 1e-5:
        assert torch.equal(idx.cpu().long(), blocks)              # block sets bit-exact
    want = oracle.attend_selected_blocks(Q, Kd, Vd, idx.cpu().long(), bs, scale)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_ragged_sequences(cuda_device):
    B, Hq, Hkv, T, bs, k = 3, 8, 2, 2048, 64, 8
    Q, K, V, _ = workloads.planted_block_cache(B, Hq, Hkv, T, seed=17)
    lens = torch.tensor([2048, 100, 1000], dtype=torch.int32)   # 100 < one k*bs window; 1000 ends mid-block
    kv, Kd, Vd = paged_case(Q, K, V, "fp8", cuda_device, seed=5, seq_lens=lens)
    meta = paged.build_block_meta(kv, bs)
    scale = 128 ** -0.5
    out, idx = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, scale, bs, k, return_indices=True)
    idx = idx.cpu().long()
    for b in range(B):
        n = int(lens[b])
        nb = (n + bs - 1) // bs
        m = oracle.block_minmax_meta(Kd[b:b + 1, :, :n], bs)
        assert torch.equal(meta[b:b + 1, :, :nb].cpu(), m)
        sc = oracle.quest_block_scores(Q[b:b + 1], m, scale)
        kk = min(k, nb)
        if score_gap(sc, kk) > 1e-5:
            assert torch.equal(idx[b:b + 1, :, :kk], oracle.topk_blocks(sc, kk))
        assert (idx[b, :, kk:] == -1).all()
    want = oracle.attend_selected_blocks(Q, Kd, Vd, idx, bs, scale, lens)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_exact_when_every_block_is_selected(cuda_device):
    """With top_k_blocks >= number of blocks the sparse path must equal dense attention."""
    Q, K, V, _ = workloads.planted_block_cache(1, 8, 2, 1024, seed=23)
    kv, Kd, Vd = paged_case(Q, K, V, "int8", cuda_device, seed=1)
    meta = paged.build_block_meta(kv, 64)
    out = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, 128 ** -0.5, 64, 16)
    want = oracle.dense_gqa_decode(Q, Kd.permute(0, 2, 1, 3), Vd.permute(0, 2, 1, 3), 128 ** -0.5)
    assert (out.float().cpu() - want).abs().max().item() <= TOL
    dense = kv.decode(Q.to(cuda_device), 128 ** -0.5)
    assert (out.float() - dense.float()).abs().max().item() <= TOL


def test_append_keeps_block_metadata_current(cuda_device):
    """Appending tokens one by one with metadata update equals rebuilding the metadata from the final cache."""
    B, Hq, Hkv, D, pages = 2, 8, 2, 128, 40
    g = torch.Generator().manual_seed(31)
    table = torch.randperm(pages, generator=g)[:B * 16].view(B, 16).to(torch.int32).to(cuda_device)
    buf = torch.zeros(pages, Hkv, paged.RECORD_ROWS, 128, dtype=torch.uint8, device=cuda_device)
    lens = torch.zeros(B, dtype=torch.int32, device=cuda_device)
    kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table, lens, B)
    meta = torch.zeros(B, Hkv, 4, 2, D, dtype=torch.float16, device=cuda_device)
    for step in range(70):   # crosses the block edge at token 64
        qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).half().to(cuda_device)
        paged.rope_quant_append(qkv, kv, Hq, 500000.0, meta=meta, block_size=64)
        lens += 1
    torch.cuda.synchronize()
    rebuilt = paged.build_block_meta(kv, 64, max_seq_len=256)
    assert torch.equal(meta[:, :, :2], rebuilt[:, :, :2])   # 70 tokens: block 0 full, block 1 holds 6 tokens


@pytest.mark.parametrize("B,Hq,Hkv,T", [(2, 32, 8, 8192), (3, 8, 2, 2048), (1, 8, 1, 131072)])
def test_ring_and_register_scoring_kernels_agree(cuda_device, lib, B, Hq, Hkv, T):
    """The block scores come from either of two kernels: metadata streamed through shared memory into tensor-core
    products with (min(q, 0) | max(q, 0)), or loaded into registers and scored with FMAs.  Both sum the same exact
    products (in different orders), so on a cache with planted high-affinity blocks they pick the same blocks and
    give the same output, also when a CTA's range crosses from one kv-head into the next and with ragged lengths."""
    Q, K, V, _ = workloads.planted_block_cache(B, Hq, Hkv, T, seed=29)
    lens = None if B == 1 else torch.tensor([T, T // 3 + 5, 70][:B], dtype=torch.int32)
    kv, Kd, Vd = paged_case(Q, K, V, "fp8", cuda_device, seed=7, seq_lens=lens)
    meta = paged.build_block_meta(kv, 64)
    res = {}
    try:
        for ring in (1, 0):
            assert lib.skv_quest_set_ring_scores(ring) == 0
            res[ring] = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, 128 ** -0.5, 64, 8, return_indices=True)
    finally:
        lib.skv_quest_set_ring_scores(1)
    assert torch.equal(res[1][1], res[0][1])
    assert torch.equal(res[1][0], res[0][0])
    want = oracle.attend_selected_blocks(Q, Kd, Vd, res[1][1].cpu().long(), 64, 128 ** -0.5, lens)
    assert (res[1][0].float().cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("B,Hq,Hkv,T,top", [(2, 32, 8, 8192, 8), (3, 8, 2, 2048, 4), (1, 8, 1, 131072, 8), (2, 6, 2, 4096, 8), (1, 4, 4, 1024, 2)])
def test_one_kernel_and_two_kernel_paths_agree(cuda_device, lib, B, Hq, Hkv, T, top):
    """The decode can run as one kernel (clusters of Hq/Hkv CTAs score a kv-head's metadata together and hand every
    head its scores through distributed shared memory); by default a scoring kernel runs first.  The scores are the
    same numbers, so blocks and outputs are identical -- for groups of 8, 4, 3 and 1 heads, ragged lengths and the
    longest sequence the fused path serves (2048 blocks)."""
    Q, K, V, _ = workloads.planted_block_cache(B, Hq, Hkv, T, seed=31)
    lens = None if B == 1 else torch.tensor([T, T // 3 + 5, 70][:B], dtype=torch.int32)
    kv, Kd, Vd = paged_case(Q, K, V, "fp8", cuda_device, seed=8, seq_lens=lens)
    meta = paged.build_block_meta(kv, 64)
    res = {}
    try:
        for fused in (1, 0):
            assert lib.skv_quest_set_fused(fused) == 0
            for _ in range(2):
                res[fused] = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, 128 ** -0.5, 64, top, return_indices=True)
            torch.cuda.synchronize()
    finally:
        lib.skv_quest_set_fused(0)
    from llm_inference_optimization_b200 import _workspace
    assert all(_workspace.status(w) == 0 for w in _workspace.all_of("quest", cuda_device))
    assert torch.equal(res[1][1], res[0][1])
    assert torch.equal(res[1][0], res[0][0])
    want = oracle.attend_selected_blocks(Q, Kd, Vd, res[1][1].cpu().long(), 64, 128 ** -0.5, lens)
    assert (res[1][0].float().cpu() - want).abs().max().item() <= TOL
