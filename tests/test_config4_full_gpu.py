"""Config 4 at full size: B=8, Hq=32, Hkv=8, D=128, 128K context, paged FP8 (page 16), block 64, top-8 blocks,
8 planted high-affinity blocks per (b, kv-head), seed 3.  The cache is built one sequence at a time (the CPU oracle
works per sequence); the kernels run once on the whole batch."""
import pytest
import torch

from llm_inference_optimization_b200 import paged, workloads
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3
B, HQ, HKV, D, T, PAGE, BS, K = 8, 32, 8, 128, 131072, 16, 64, 8


def test_quest_decode_config4_full_size(cuda_device, record_property):
    pps = T // PAGE
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(B * pps, generator=g)
    buf = torch.zeros(B * pps, HKV, paged.RECORD_ROWS, 128, dtype=torch.uint8, device=cuda_device)
    kp, vp, ksp, vsp = paged.fused_views(buf, torch.float8_e4m3fn)
    table = perm.view(B, pps).to(torch.int32)
    Qs, metas, deq, planted = [], [], [], []
    for b in range(B):
        Q, Kb, Vb, ids = workloads.planted_block_cache(1, HQ, HKV, T, seed=3 + 17 * b)
        kc, ks = oracle.quantize_e4m3(Kb)
        vc, vs = oracle.quantize_e4m3(Vb)
        pg = table[b].long().to(cuda_device)
        # [1,Hkv,T,D] -> [pps,Hkv,16,D] rows of this sequence's pages
        kp.view(torch.uint8)[pg] = kc.view(torch.uint8).view(HKV, pps, PAGE, D).permute(1, 0, 2, 3).contiguous().to(cuda_device)
        vp.view(torch.uint8)[pg] = vc.view(torch.uint8).view(HKV, pps, PAGE, D).permute(1, 0, 2, 3).contiguous().to(cuda_device)
        ksp[pg] = ks.view(HKV, pps, PAGE).permute(1, 0, 2).contiguous().to(cuda_device)
        vsp[pg] = vs.view(HKV, pps, PAGE).permute(1, 0, 2).contiguous().to(cuda_device)
        Kd = oracle.dequantize(kc, ks)
        metas.append(oracle.block_minmax_meta(Kd, BS))
        # keep only what the output check needs: dequantised K/V are re-derived per selected block below
        deq.append((kc, ks, vc, vs))
        Qs.append(Q)
        planted.append(ids)
        del Kb, Vb, Kd
    Q = torch.cat(Qs)
    kv = paged.PagedKV(kp, vp, ksp, vsp, table.to(cuda_device), None, B)
    scale = D ** -0.5

    meta = paged.build_block_meta(kv, BS)
    want_meta = torch.cat(metas)
    assert torch.equal(meta.cpu(), want_meta)                                   # metadata bit-exact at full size

    out, idx = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, scale, BS, K, return_indices=True)
    idx = idx.cpu().long()
    sc = oracle.quest_block_scores(Q, want_meta, scale)
    top = sc.topk(K + 1, -1).values
    clear = (top[..., K - 1] - top[..., K]) > 1e-5                             # heads whose k-th boundary is not a near tie
    want_blocks = oracle.topk_blocks(sc, K)
    assert clear.float().mean().item() > 0.9
    assert torch.equal(idx[clear], want_blocks[clear])                          # block sets bit-exact

    # exact attention over the selected blocks, per sequence (only 8 x 64 tokens per head are touched)
    for b in range(B):
        kc, ks, vc, vs = deq[b]
        tok = (idx[b].view(HQ, K, 1) * BS + torch.arange(BS).view(1, 1, BS)).view(HQ, K * BS)
        for hq in range(HQ):
            h = hq // (HQ // HKV)
            kk = kc[0, h, tok[hq]].float() * ks[0, h, tok[hq]].unsqueeze(-1)
            vv = vc[0, h, tok[hq]].float() * vs[0, h, tok[hq]].unsqueeze(-1)
            p = torch.softmax((kk @ Q[b, hq].float()) * scale, 0)
            assert (out[b, hq].float().cpu() - p @ vv).abs().max().item() <= TOL

    # report (not a gate): how many planted blocks each scoring rule recovers on this synthetic data
    hits = 0
    for b in range(B):
        for hq in range(HQ):
            hits += len(set(idx[b, hq].tolist()) & set(planted[b][0, hq // (HQ // HKV)].tolist()))
    record_property("planted_block_recall_minmax_rule", hits / (B * HQ * K))
    print(f"planted-block recall of the min/max upper-bound rule: {hits / (B * HQ * K):.3f}")


def test_block_mean_rule_recovers_planted_blocks_at_128k(cuda_device, record_property):
    """The reference's block-mean rule on the same synthetic data (one sequence, heads expanded as the reference's
    caller does with repeat_kv): block sets equal the oracle's and contain the planted blocks."""
    from llm_inference_optimization_b200 import _C
    Q, Kb, Vb, ids = workloads.planted_block_cache(1, HQ, HKV, T, seed=3)
    G = HQ // HKV
    Kx = Kb.repeat_interleave(G, dim=1)   # [1,Hq,T,D] fp16
    Vx = Vb.repeat_interleave(G, dim=1)
    Q4 = Q.unsqueeze(2)                   # [1,Hq,1,D]
    out, idx = _C.sparse_attention_forward(Q4.to(cuda_device), Kx.to(cuda_device), Vx.to(cuda_device), BS, K,
                                           return_indices=True)
    want, blocks = oracle.block_sparse_mean_attention(Q4, Kx, Vx, BS, K)
    assert torch.equal(idx.cpu().long(), blocks)
    assert (out.float().cpu() - want).abs().max().item() <= TOL
    hits = sum(len(set(idx[0, hq].tolist()) & set(ids[0, hq // G].tolist())) for hq in range(HQ))
    record_property("planted_block_recall_mean_rule", hits / (HQ * K))
    print(f"planted-block recall of the block-mean rule: {hits / (HQ * K):.3f}")
    assert hits == HQ * K
