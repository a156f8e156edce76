"""Host logic of the tensor-parallel decode step on CPU: sharding maps, and world_size-2 gloo ranks whose
summed partial results must equal the single-rank model.  The attention kernel is replaced by the oracle here
(the product default stays the CUDA kernel); everything else is the product code path."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llm_inference_optimization_b200 import decode_step as ds
from llm_inference_optimization_b200.sharding import shard_columns, shard_heads
from oracle import skv_oracle as oracle

CFG = ds.ModelConfig(layers=2, hidden=256, Hq=8, Hkv=4, D=128, mlp=512, vocab=320)
LENS = torch.tensor([37, 5, 64], dtype=torch.int32)


def oracle_attention(q, cache, page_table, seq_lens, scale, max_seq_len):
    """Dense decode over the dequantised pages of a LayerCache, by the CPU oracle."""
    B = q.shape[0]
    n_kv = cache.k.shape[1]
    T = page_table.shape[1] * 16
    K = torch.zeros(B, T, n_kv, 128)
    V = torch.zeros(B, T, n_kv, 128)
    for b in range(B):
        pg = page_table[b].long()
        K[b] = oracle.dequantize(cache.k[pg], cache.ks[pg]).permute(0, 2, 1, 3).reshape(T, n_kv, 128)
        V[b] = oracle.dequantize(cache.v[pg], cache.vs[pg]).permute(0, 2, 1, 3).reshape(T, n_kv, 128)
    return oracle.dense_gqa_decode(q.half().float(), K, V, scale, seq_lens)


def test_head_sharding_maps():
    s = shard_heads(32, 8, 4, 2)
    assert list(s.kv_heads) == [4, 5] and list(s.q_heads) == list(range(16, 24))
    assert all(q // 4 in s.kv_heads for q in s.q_heads)
    covered = [h for r in range(8) for h in shard_heads(32, 8, 8, r).kv_heads]
    assert covered == list(range(8))
    assert list(shard_columns(14336, 8, 7)) == list(range(12544, 14336))
    with pytest.raises(ValueError):
        shard_heads(32, 8, 3, 0)
    with pytest.raises(ValueError):
        shard_heads(30, 8, 2, 0)


def single_rank_logits(steps=2):
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), "cpu", dtype=torch.float32, attention=oracle_attention)
    m.init_cache(LENS)
    tok = torch.tensor([3, 100, 250])
    outs = []
    for _ in range(steps):
        logits = m.step(tok)
        outs.append(logits)
        tok = logits.argmax(-1)
    return outs, m


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, world, rank), "cpu", dtype=torch.float32,
                           attention=oracle_attention)
        m.init_cache(LENS)
        tok = torch.tensor([3, 100, 250])
        outs = []
        for _ in range(2):
            logits = m.step(tok)
            outs.append(logits)
            tok = logits.argmax(-1)
        if rank == 0:
            ret.put([o.numpy() for o in outs])
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_single_rank():
    want, _ = single_rank_logits()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = ret.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for g, w in zip(got, want):
        assert torch.allclose(torch.from_numpy(g), w, atol=2e-4, rtol=1e-4)


def test_single_rank_matches_fp32_oracle_model():
    """The whole step (norms, RoPE, append-quantise, attention, MLP) vs the independent fp32 restatement."""
    from oracle import decode_step_oracle as dso
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), "cpu", dtype=torch.float32, attention=oracle_attention)
    m.init_cache(LENS)
    B, T = LENS.numel(), m.page_table.shape[1] * 16
    k_hist, v_hist = [], []
    for c in m.caches:
        K = torch.zeros(B, CFG.Hkv, T, 128)
        V = torch.zeros(B, CFG.Hkv, T, 128)
        for b in range(B):
            pg = m.page_table[b].long()
            K[b] = oracle.dequantize(c.k[pg], c.ks[pg]).permute(1, 0, 2, 3).reshape(CFG.Hkv, T, 128)
            V[b] = oracle.dequantize(c.v[pg], c.vs[pg]).permute(1, 0, 2, 3).reshape(CFG.Hkv, T, 128)
        k_hist.append(K)
        v_hist.append(V)
    D = CFG.D
    weights = {"embed": m.embed, "lm_head": m.lm_head, "final_norm": m.final_norm, "layers": []}
    for w in m.layers:
        nq, nk = CFG.Hq * D, CFG.Hkv * D
        half = w["wgu"].shape[1] // 2
        weights["layers"].append(dict(wq=w["wqkv"][:, :nq], wk=w["wqkv"][:, nq:nq + nk], wv=w["wqkv"][:, nq + nk:],
                                      wo=w["wo"], wg=w["wgu"][:, :half], wu=w["wgu"][:, half:], wd=w["wd"],
                                      n1=w["n1"], n2=w["n2"]))
    tok = torch.tensor([3, 100, 250])
    want = dso.decode_step(weights, CFG, tok, k_hist, v_hist, LENS.clone())
    got = m.step(tok)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4)
    assert torch.equal(m.seq_lens.cpu(), LENS + 1)
