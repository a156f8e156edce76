"""Throughput of the full tensor-parallel decode step (random-init Llama-3.1-8B architecture, FP8 paged KV).

    python -m llm_inference_optimization_b200.bench_decode [--steps 20] [--warmup 3] [--layers 32]
    python -m torch.distributed.run --nproc-per-node N -m llm_inference_optimization_b200.bench_decode ...

Batch 16, context lengths uniform in [8K, 128K] (seed 4), one decode step captured in a CUDA graph and
replayed; tokens/s = batch / step time (max over ranks).  The reference times the same step on its patched
Hugging Face model with ``time.perf_counter`` (benchmarks/llama_integration_benchmark.py:266-279).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import decode_step as ds
from .sharding import shard_heads


def ideal_bytes(cfg: ds.ModelConfig, lens: torch.Tensor, world: int) -> dict:
    per_layer_w = cfg.hidden * (cfg.Hq + 2 * cfg.Hkv) * cfg.D + cfg.Hq * cfg.D * cfg.hidden + 3 * cfg.hidden * cfg.mlp
    head = cfg.hidden * cfg.vocab / (world if cfg.vocab % world == 0 else 1)        # split by vocabulary columns
    weights = 2 * (cfg.layers * per_layer_w / world + head)                         # bf16
    kv = int(lens.sum()) * cfg.layers * 2 * (cfg.Hkv // world) * (cfg.D + 4)        # fp8 codes + fp32 scales
    return {"weight_bytes_per_gpu": int(weights), "kv_bytes_per_gpu": int(kv)}


PARITY_CFG = ds.ModelConfig(layers=2, hidden=1024, Hq=32, Hkv=8, D=128, mlp=2048, vocab=1024)
PARITY_TOL = {"max_abs_over_logit_scale": 3e-2, "cos_min": 0.999}


def tp_parity(world: int, rank: int, dev, fused_allreduce: bool) -> dict | None:
    """Tensor-parallel ranks against one rank, on real GPUs, before anything is timed.

    A 2-layer model of reduced width (same head layout, so it shards over up to 8 ranks) takes one decode step on
    all ranks with the all-reduce the benchmark uses, and on rank 0 alone as a single-rank model built from the same
    full weights and cache bytes.  bf16 sums in a different order: the logits must agree to a few percent of the
    logit scale.  Raises on rank 0 (after every rank has left the collective calls) when they do not."""
    cfg = PARITY_CFG
    lens = torch.tensor([700, 37, 100, 1500], dtype=torch.int32)
    tok = torch.tensor([3, 100, 250, 999], device=dev)
    m = ds.DecodeModel(cfg, shard_heads(cfg.Hq, cfg.Hkv, world, rank), dev, seed=11)
    m.init_cache(lens, fill="normal", seed=11)
    if fused_allreduce:   # every rank takes the same path: NCCL for all when one of them cannot set the kernel up
        try:
            m.enable_fused_allreduce(lens.numel())
            ok = 1
        except Exception:  # noqa: BLE001
            ok = 0
        agree = torch.tensor([ok], device=dev, dtype=torch.int32)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        fused_allreduce = bool(int(agree.item()))
        m.fused_allreduce = fused_allreduce
    got = m.step(tok).float()
    torch.cuda.synchronize()
    dist.barrier()
    res = None
    if rank == 0:
        single = ds.DecodeModel(cfg, shard_heads(cfg.Hq, cfg.Hkv, 1, 0), dev, seed=11)
        single.init_cache(lens, fill="normal", seed=11)
        want = single.step(tok).float()
        scale = max(1e-6, want.abs().max().item())
        res = {"world": world, "max_abs": (got - want).abs().max().item(), "logit_scale": scale,
               "cos_min": torch.nn.functional.cosine_similarity(got, want, dim=-1).min().item(),
               "tol": PARITY_TOL, "all_reduce": "fused peer-memory kernel" if fused_allreduce else "nccl",
               "model": "2 layers, hidden 1024, 32/8 heads, bf16, FP8 paged cache"}
        del single
    del m
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    dist.barrier()
    if res is not None and (res["max_abs"] > PARITY_TOL["max_abs_over_logit_scale"] * res["logit_scale"]
                            or res["cos_min"] < PARITY_TOL["cos_min"]):
        raise RuntimeError(f"tensor-parallel logits differ from the single-rank model: {res}")
    return res


def run(steps: int = 20, warmup: int = 3, layers: int = 32, batch: int = 16, seed: int = 4, use_graph: bool = True,
        fill: str = "random_codes", fused_allreduce: bool = True, hybrid_dense_layers: int | None = None,
        emulate_tp: int = 0, mixed_pages: bool = False) -> dict | None:
    """``emulate_tp`` (single process only): build rank 0's shard of an ``emulate_tp``-way tensor-parallel model on one
    GPU and run its step without the exchange -- every kernel then has the shapes it has at that degree, which is what
    a per-kernel launch list needs (a profiler must not wrap a multi-rank run).  ``mixed_pages``: afterwards the same
    step is timed over caches of mixed-precision page records (FP8 keys, 4-bit values)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    parity = None
    if world > 1:
        # with the all-reduce the timed run uses (the fused kernel when this machine offers symmetric memory)
        parity = tp_parity(world, rank, dev, fused_allreduce)
    cfg = ds.ModelConfig(layers=layers)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(8192, 131073, (batch,), generator=g, dtype=torch.int32)
    shard_world = emulate_tp if (emulate_tp > 1 and world == 1) else world
    model = ds.DecodeModel(cfg, shard_heads(cfg.Hq, cfg.Hkv, shard_world, rank), dev, seed=seed)
    if shard_world != world:
        model._all_reduce = lambda x: x   # one rank of the emulated group: its partial sums stand in for the reduced ones
        model._all_gather_columns = lambda x: x   # ... and its slice of the logits for all of them
    model.init_cache(lens, fill=fill, seed=seed, extra_tokens=2 * (steps + warmup) + 32)
    fused_allreduce = fused_allreduce and world > 1
    if fused_allreduce:
        # all-reduce + residual + RMSNorm in one peer-memory kernel, no NCCL call; if the symmetric-memory
        # rendezvous is not available on this machine every rank falls back to NCCL all-reduces together
        try:
            model.enable_fused_allreduce(batch)
            ok = 1
        except Exception as e:  # noqa: BLE001 -- reported below, the NCCL path still measures the step
            print(f"[bench_decode] rank {rank}: fused all-reduce unavailable ({type(e).__name__}: {e})", flush=True)
            ok = 0
        agree = torch.tensor([ok], device=dev, dtype=torch.int32)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            model.fused_allreduce = False
            fused_allreduce = False
    tok = torch.randint(0, cfg.vocab, (batch,), generator=g).to(dev)

    def timed_run():
        """Warm up, capture one step in a CUDA graph (optional), replay it `steps` times; ms per step, max over ranks."""
        logits = None
        for _ in range(warmup):
            logits = model.step(tok)
        torch.cuda.synchronize()
        graph = None
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                model.step(tok)  # once on the capture stream so that its workspaces exist
            torch.cuda.current_stream().wait_stream(side)
            with torch.cuda.graph(graph):
                logits = model.step(tok)
            step = graph.replay
        else:
            holder = {}

            def step():
                holder["logits"] = model.step(tok)
        step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms_ = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms_], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_ = float(t.item())
        if not use_graph:
            logits = holder["logits"]
        fin = bool(torch.isfinite(logits.float()).all().item())
        # the captured graph holds NCCL kernels: release it before anybody tears the communicator down
        step = None
        del graph
        torch.cuda.synchronize()
        return ms_, fin

    ms, finite = timed_run()

    hybrid = None
    if hybrid_dense_layers is not None and 0 <= hybrid_dense_layers < layers:
        # The reference's layer sweep (results/llama_run_20260628_233732/layer_sweep.json:20-37): sparse attention in
        # some layers only.  Same token, same cache, dense schedule against the hybrid one, then the hybrid step timed.
        saved = model.seq_lens.clone()
        logits_dense = model.step(tok).float()
        model.seq_lens.copy_(saved)
        modes = ["dense"] * hybrid_dense_layers + ["quest"] * (layers - hybrid_dense_layers)
        model.set_layer_modes(modes)
        logits_hybrid = model.step(tok).float()
        drift = (logits_hybrid - logits_dense).abs()
        match = (logits_hybrid.argmax(-1) == logits_dense.argmax(-1)).float().mean()
        ms_h, fin_h = timed_run()
        hybrid = {"dense_layers": hybrid_dense_layers, "sparse_layers": layers - hybrid_dense_layers,
                  "sparse_rule": f"Quest min/max bound, top {model.quest_top_k} blocks of {model.quest_block} tokens per query head",
                  "ms_per_step": ms_h, "value": batch / (ms_h * 1e-3), "unit": "tok/s", "logits_finite": fin_h,
                  "speedup_vs_all_dense": ms / ms_h,
                  "mean_abs_logit_diff_vs_all_dense": float(drift.mean().item()),
                  "max_abs_logit_diff_vs_all_dense": float(drift.max().item()),
                  "argmax_match_vs_all_dense": float(match.item()),
                  "note": "random-init weights and a random cache: the drift says what the schedule does to THESE logits, "
                          "not what it does to a trained model"}
        model.set_layer_modes(None)
    if fused_allreduce and model.arn.status() != 0:
        raise RuntimeError("a bounded wait for a peer ran out inside the fused all-reduce kernel")
    mixed = None
    if mixed_pages:
        # the same model, lengths and page tables over mixed-precision page records: 200 instead of 264 bytes per token
        # and kv-head (the first model's caches are freed first: the two do not fit side by side at every size)
        del model
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        model = ds.DecodeModel(cfg, shard_heads(cfg.Hq, cfg.Hkv, shard_world, rank), dev, seed=seed, v_bits=4)
        if shard_world != world:
            model._all_reduce = lambda x: x
            model._all_gather_columns = lambda x: x
        model.init_cache(lens, fill=fill, seed=seed, extra_tokens=2 * (steps + warmup) + 32)
        if fused_allreduce:
            model.enable_fused_allreduce(batch)
        ms_m, fin_m = timed_run()
        if fused_allreduce and model.arn.status() != 0:
            raise RuntimeError("a bounded wait for a peer ran out inside the fused all-reduce kernel")
        mixed = {"kv": "FP8-E4M3 keys, 4-bit values (mixed-precision page records), " + fill, "ms_per_step": ms_m,
                 "value": batch / (ms_m * 1e-3), "unit": "tok/s", "logits_finite": fin_m, "speedup_vs_fp8_values": ms / ms_m,
                 "kv_bytes_per_gpu": ideal_bytes(cfg, lens, shard_world)["kv_bytes_per_gpu"] * 200 // 264}
        if hybrid is not None:   # both together: the hybrid schedule over the mixed-precision caches
            model.set_layer_modes(["dense"] * hybrid_dense_layers + ["quest"] * (layers - hybrid_dense_layers))
            ms_mh, fin_mh = timed_run()
            mixed["hybrid_schedule"] = {"ms_per_step": ms_mh, "value": batch / (ms_mh * 1e-3), "unit": "tok/s",
                                        "logits_finite": fin_mh, "speedup_vs_all_dense_fp8_values": ms / ms_mh}
    ib = ideal_bytes(cfg, lens, shard_world)
    out = {
        "metric": "decode_step_tokens_per_s", "value": batch / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms,
        "n_gpus": world, "emulated_tp_shard": shard_world if shard_world != world else None, "steps": steps, "warmup": warmup, "cuda_graph": use_graph, "logits_finite": finite,
        "tp_parity": parity, "hybrid_schedule": hybrid, "mixed_precision_pages": mixed,
        "config": {"model": "Llama-3.1-8B architecture, random init N(0,0.02), bf16 weights", "layers": layers,
                   "batch": batch, "context_lengths": "uniform 8192..131072, seed 4", "total_context_tokens": int(lens.sum()),
                   "kv": "FP8-E4M3 paged (page 16, fused page records), per-token-per-head fp32 scales, " + fill,
                   "parallelism": f"tp{world} by KV head, " + (
                       "all-reduce after o_proj and down_proj fused with residual + RMSNorm over NVLink peer memory"
                       if fused_allreduce else "NCCL all-reduce after o_proj and down_proj")},
        **ib,
        "hbm_bytes_per_step_per_gpu": ib["weight_bytes_per_gpu"] + ib["kv_bytes_per_gpu"],
        "achieved_GBps_per_gpu": (ib["weight_bytes_per_gpu"] + ib["kv_bytes_per_gpu"]) / (ms * 1e-3) / 1e9,
    }
    del model
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return out if rank == 0 else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--nccl-allreduce", action="store_true", help="use NCCL all-reduces instead of the fused kernel")
    ap.add_argument("--emulate-tp", type=int, default=0,
                    help="single process: run rank 0's shard of an N-way tensor-parallel model without the exchange")
    ap.add_argument("--hybrid-dense-layers", type=int, default=None,
                    help="also time a schedule with dense attention in the first N layers and Quest block-sparse attention in the rest")
    ap.add_argument("--mixed-pages", action="store_true",
                    help="also time the step over mixed-precision page records (FP8 keys, 4-bit values)")
    args = ap.parse_args()
    res = run(args.steps, args.warmup, args.layers, args.batch, use_graph=not args.no_graph,
              fused_allreduce=not args.nccl_allreduce, hybrid_dense_layers=args.hybrid_dense_layers,
              emulate_tp=args.emulate_tp, mixed_pages=args.mixed_pages)
    if res is not None:
        print(json.dumps(res), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
