"""The full decode step on the GPU (paged FP8 cache, sm_100a attention kernel) vs the fp32 CPU oracle model,
and tensor-parallel ranks vs a single rank when more than one GPU is present."""
import os
import socket

import pytest
import torch

from llm_inference_optimization_b200 import decode_step as ds
from llm_inference_optimization_b200.sharding import shard_heads
from oracle import decode_step_oracle as dso
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
CFG = ds.ModelConfig(layers=2, hidden=512, Hq=8, Hkv=2, D=128, mlp=1024, vocab=512)
LENS = torch.tensor([100, 37, 700], dtype=torch.int32)
TOK = torch.tensor([3, 100, 250])


def oracle_inputs(m):
    B, T = LENS.numel(), m.page_table.shape[1] * 16
    pt = m.page_table.cpu()
    k_hist, v_hist = [], []
    for c in m.caches:
        k, v, ks, vs = (t.cpu() for t in (c.k, c.v, c.ks, c.vs))
        K = torch.zeros(B, CFG.Hkv, T, 128)
        V = torch.zeros(B, CFG.Hkv, T, 128)
        for b in range(B):
            pg = pt[b].long()
            K[b] = oracle.dequantize(k[pg], ks[pg]).permute(1, 0, 2, 3).reshape(CFG.Hkv, T, 128)
            V[b] = oracle.dequantize(v[pg], vs[pg]).permute(1, 0, 2, 3).reshape(CFG.Hkv, T, 128)
        k_hist.append(K)
        v_hist.append(V)
    D = CFG.D
    weights = {"embed": m.embed.float().cpu(), "lm_head": m.lm_head.float().cpu(), "final_norm": m.final_norm.float().cpu(),
               "layers": []}
    for w in m.layers:
        w = {k: v.float().cpu() for k, v in w.items()}
        nq, nk = CFG.Hq * D, CFG.Hkv * D
        half = w["wgu"].shape[1] // 2
        weights["layers"].append(dict(wq=w["wqkv"][:, :nq], wk=w["wqkv"][:, nq:nq + nk], wv=w["wqkv"][:, nq + nk:],
                                      wo=w["wo"], wg=w["wgu"][:, :half], wu=w["wgu"][:, half:], wd=w["wd"],
                                      n1=w["n1"], n2=w["n2"]))
    return weights, k_hist, v_hist


def test_fp32_weights_match_oracle_model(cuda_device):
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.float32)
    m.init_cache(LENS)
    weights, k_hist, v_hist = oracle_inputs(m)
    want = dso.decode_step(weights, CFG, TOK, k_hist, v_hist, LENS.clone())
    got = m.step(TOK.to(cuda_device)).cpu()
    assert torch.equal(m.seq_lens.cpu(), LENS + 1)
    assert (got - want).abs().max().item() <= 5e-3 * max(1.0, want.abs().max().item())


def test_bf16_weights_and_cuda_graph_replay(cuda_device):
    ref = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.float32)
    ref.init_cache(LENS)
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16)
    m.init_cache(LENS)
    tok = TOK.to(cuda_device)
    want = ref.step(tok)
    got = m.step(tok).float()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert cos.min().item() > 0.995
    # second token through a captured graph equals the eager second token
    m2 = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16)
    m2.init_cache(LENS)
    m2.step(tok)
    eager = m.step(tok).float()
    graph = torch.cuda.CUDAGraph()
    static_tok = tok.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        saved = m2.seq_lens.clone()
        m2.step(static_tok)              # warm-up on the side stream (allocates workspaces)
        m2.seq_lens.copy_(saved)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(graph):
        out = m2.step(static_tok)
    m2.seq_lens.copy_(saved)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), eager, atol=2e-2, rtol=2e-2)
    assert torch.equal(m2.seq_lens.cpu(), LENS + 2)


def _tp_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, world, rank), torch.device("cuda", rank), dtype=torch.float32)
        m.init_cache(LENS)
        out = m.step(TOK.cuda())
        if rank == 0:
            ret.put(out.cpu().numpy())
    finally:
        dist.destroy_process_group()


def test_two_gpu_tensor_parallel_matches_single(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    single = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.float32)
    single.init_cache(LENS)
    want = single.step(TOK.to(cuda_device)).cpu()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = torch.from_numpy(ret.get(timeout=300))
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert torch.allclose(got, want, atol=2e-3, rtol=1e-3)
