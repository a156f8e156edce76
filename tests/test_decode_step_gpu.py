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
            vd = oracle.dequantize_int4(v[pg], vs[pg]) if c.v_bits == 4 else oracle.dequantize(v[pg], vs[pg])
            V[b] = vd.permute(1, 0, 2, 3).reshape(CFG.Hkv, T, 128)
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


def test_bf16_fused_glue_path_matches_oracle_model(cuda_device):
    """The path the decode benchmark times -- bf16 weights, fused RoPE/quantise/append, residual-RMSNorm and SiLU
    kernels, bf16 attention output -- against the fp32 CPU oracle evaluated on the same (bf16-rounded) weights."""
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16)
    assert m.fused_glue
    m.init_cache(LENS)
    weights, k_hist, v_hist = oracle_inputs(m)            # .float() of bf16 tensors: the rounded weights themselves
    want = dso.decode_step(weights, CFG, TOK, k_hist, v_hist, LENS.clone())
    got = m.step(TOK.to(cuda_device)).float().cpu()
    err = (got - want).abs().max().item()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1).min().item()
    print(f"bf16 fused-glue step vs fp32 oracle: max-abs {err:.3e} (logits up to {want.abs().max().item():.3f}), cos {cos:.6f}")
    # bf16 activations carry 8 mantissa bits through two layers: a few 1e-3 of the logit scale
    assert err <= 2e-2 * max(1.0, want.abs().max().item())
    assert cos > 0.999


def test_weight_streaming_gemm_option_matches_oracle_model(cuda_device):
    """skinny_gemm=True routes the four projections of every layer through this library's GEMM kernel."""
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16, skinny_gemm=True)
    m.init_cache(LENS)
    weights, k_hist, v_hist = oracle_inputs(m)
    want = dso.decode_step(weights, CFG, TOK, k_hist, v_hist, LENS.clone())
    got = m.step(TOK.to(cuda_device)).float().cpu()
    from llm_inference_optimization_b200 import _workspace
    assert _workspace.all_of("skinny_gemm", cuda_device), "the weight-streaming kernel did not run"
    assert (got - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
    assert torch.nn.functional.cosine_similarity(got, want, dim=-1).min().item() > 0.999


def test_mixed_precision_pages_match_oracle_model(cuda_device):
    """v_bits=4: FP8 keys and 4-bit values in every layer's cache -- appended by the fused kernel, read by the decode
    kernel's 4-bit path -- against the oracle model that stores the new value row by the same 4-bit rule."""
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16, v_bits=4)
    m.init_cache(LENS)
    assert m.caches[0].buf.shape[2] == 25
    weights, k_hist, v_hist = oracle_inputs(m)
    want = dso.decode_step(weights, CFG, TOK, k_hist, v_hist, LENS.clone(), v_bits=4)
    got = m.step(TOK.to(cuda_device)).float().cpu()
    assert (got - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
    assert torch.nn.functional.cosine_similarity(got, want, dim=-1).min().item() > 0.999
    with pytest.raises(ValueError):   # block-sparse layers over 4-bit values gather at most 512 tokens
        ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16, v_bits=4,
                       layer_modes=["dense", "quest"], quest_block=64, quest_top_k=16)


def test_hybrid_schedule_over_mixed_precision_pages_matches_oracle_model(cuda_device):
    """Dense layer 0, Quest block-sparse layer 1, both over FP8 keys and 4-bit values."""
    modes = ["dense", "quest"]
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.float32, layer_modes=modes,
                       quest_block=16, quest_top_k=3, v_bits=4)
    m.init_cache(LENS)
    weights, k_hist, v_hist = oracle_inputs(m)
    want = dso.decode_step(weights, CFG, TOK, k_hist, v_hist, LENS.clone(), layer_modes=modes, quest_block=16,
                           quest_top_k=3, v_bits=4)
    got = m.step(TOK.to(cuda_device)).cpu()
    assert (got - want).abs().max().item() <= 5e-3 * max(1.0, want.abs().max().item())


def test_hybrid_layer_schedule_matches_oracle_model(cuda_device):
    """Dense attention in layer 0, Quest block-sparse attention (4 blocks of 64 tokens) in layer 1, against the oracle
    model with the same schedule."""
    modes = ["dense", "quest"]
    m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.float32, layer_modes=modes,
                       quest_block=64, quest_top_k=4)
    m.init_cache(LENS)
    weights, k_hist, v_hist = oracle_inputs(m)
    want = dso.decode_step(weights, CFG, TOK, k_hist, v_hist, LENS.clone(), layer_modes=modes, quest_block=64, quest_top_k=4)
    dense = dso.decode_step(weights, CFG, TOK, k_hist, v_hist, LENS.clone())
    got = m.step(TOK.to(cuda_device)).cpu()
    assert (got - want).abs().max().item() <= 5e-3 * max(1.0, want.abs().max().item())
    assert (want - dense).abs().max().item() > 1e-3      # the schedule really changes the longest sequence's result


def test_sparse_layers_that_select_every_block_equal_the_dense_model(cuda_device):
    """The benchmarked path (bf16, fused glue kernels) with every layer block-sparse and top_k covering the whole
    cache must reproduce the all-dense model, also on the second token, whose blocks' metadata was brought up to
    date by the append kernel rather than rebuilt."""
    tok = TOK.to(cuda_device)
    dense = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16)
    dense.init_cache(LENS)
    sparse = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, 1, 0), cuda_device, dtype=torch.bfloat16,
                            layer_modes=["quest", "quest"], quest_block=64, quest_top_k=16)
    sparse.init_cache(LENS)
    for _ in range(2):
        want, got = dense.step(tok).float(), sparse.step(tok).float()
        assert (got - want).abs().max().item() <= 3e-2 * max(1.0, want.abs().max().item())
    # switching a layer back to dense and then to sparse again rebuilds its metadata instead of reusing a stale one
    sparse.set_layer_modes(["dense", "quest"])
    dense.step(tok), sparse.step(tok)
    sparse.set_layer_modes(["quest", "quest"])
    want, got = dense.step(tok).float(), sparse.step(tok).float()
    assert (got - want).abs().max().item() <= 3e-2 * max(1.0, want.abs().max().item())


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


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("code_dtype", [torch.int8, torch.float8_e4m3fn])
def test_rope_quant_append_kernel(cuda_device, dtype, code_dtype):
    """The one-launch RoPE + quantise + append against an fp32 restatement of the same three steps."""
    from llm_inference_optimization_b200 import paged
    B, Hq, Hkv, D, pages = 3, 8, 2, 128, 64
    g = torch.Generator().manual_seed(12)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    lens = torch.tensor([0, 17, 255], dtype=torch.int32)
    table = torch.randperm(pages, generator=g)[:B * 16].view(B, 16).to(torch.int32)
    buf = torch.zeros(pages, Hkv, paged.RECORD_ROWS, 128, dtype=torch.uint8, device=cuda_device)
    kv = paged.PagedKV.from_fused(buf, code_dtype, table.to(cuda_device), lens.to(cuda_device), B)
    q = paged.rope_quant_append(qkv.to(cuda_device), kv, Hq, 500000.0).float().cpu()
    x = qkv.float().view(B, Hq + 2 * Hkv, D)
    want_q = dso.rope(x[:, :Hq], lens, 500000.0)          # the oracle's restatement, not the package's own function
    want_k = dso.rope(x[:, Hq:Hq + Hkv], lens, 500000.0)
    want_v = x[:, Hq + Hkv:]
    assert (q - want_q).abs().max().item() <= 4e-3
    quant = oracle.quantize_int8 if code_dtype == torch.int8 else oracle.quantize_e4m3
    for pool, spool, want in ((kv.k_pool, kv.k_scale, want_k), (kv.v_pool, kv.v_scale, want_v)):
        for b in range(B):
            page, slot = int(table[b, int(lens[b]) // 16]), int(lens[b]) % 16
            codes, scale = pool[page, :, slot].cpu(), spool[page, :, slot].cpu()
            wc, ws = quant(want[b])
            assert torch.allclose(scale, ws, rtol=1e-5)
            if code_dtype == torch.int8:
                assert (codes.int() - wc.int()).abs().max().item() <= 1   # sin/cos differ in the last ulp
            else:
                assert oracle.e4m3_code_distance(codes, wc).max().item() <= 1
    # nothing else in the pool was touched
    touched = torch.zeros(pages, dtype=torch.bool)
    for b in range(B):
        touched[int(table[b, int(lens[b]) // 16])] = True
    assert (buf.cpu()[~touched] == 0).all()
