#!/usr/bin/env python
"""Benchmark of the dense GQA decode-attention hot path (the metric the baseline is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--ctx 65536]

Workload ("config 2", Llama-3.1-8B layer shape): B=1 per GPU-share, Hq=32, Hkv=8, D=128, fp16 KV
cache of `ctx` tokens in the reference's [B, N, Hkv, D] layout, one query token.  One STEP is one
decode pass over the attention of a 32-layer model: 32 launches of the decode kernel, each over
its own layer's KV cache (32 x 268 MB at 64K, so consecutive launches never find their input in
the 126 MB L2).  `value` is KV bytes streamed per second (GB/s) with the caches resident in HBM and
launches in the library's default order (each launch waits for the one before, as it must inside a
real decode step); `us_per_layer` is the same time divided by 32.

With N > 1 GPUs the path is partitioned by KV head and needs no collective: rank r owns
Hkv / N kv-heads (and their 4 query heads each) of N sequences, so the work per GPU stays that
of one sequence ("weak" scaling) while the global batch grows with N.

`--impl reference` times the reference's CPU check of this path (fp32 softmax(QK^T)V over
repeat_kv-expanded heads, restated in oracle/) on all host cores: same workload description, the
same number of warm-up and timed steps, every step really run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = 32
HQ, HKV, D = 32, 8, 128
FALLBACK_HBM_GBS = 6650.0
METRIC = "decode_attn_kv_stream_bandwidth"
DTYPE = "f16 storage, f32 accumulate"
# DRAM bytes one launch of the decode kernel moves at context 65536 (dram__bytes_read.sum + dram__bytes_write.sum of one
# ncu capture of gqa_decode_f16_kernel<128>); other contexts report null.
NCU_TRAFFIC_BYTES_64K = 271_700_000


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def workload_config(ctx: int, layers: int, world: int) -> dict:
    """The workload both arms run; identical dictionaries so the two JSON lines can be compared key by key."""
    per_layer = kv_bytes(ctx, HKV // world, world)
    return {
        "workload": f"config2 dense GQA decode, Llama-3.1-8B layer shape, context {ctx}, {layers} layers per step",
        "global_batch": world, "Hq": HQ, "Hkv": HKV, "D": D, "ctx": ctx, "layers_per_step": layers,
        "partition": f"kv-head: {HKV // world} kv-heads x {world} sequences per GPU, no collective",
        "l2": f"inputs larger than L2: each layer pass reads its own {per_layer / 1e6:.0f} MB cache per GPU",
    }


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML while the timed region runs."""

    def __init__(self, torch_index: int):
        self.samples, self.reasons, self.err = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            pr = torch.cuda.get_device_properties(torch_index)
            bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report, do not fail the bench
            self.err = f"{type(e).__name__}: {e}"

    def _once(self):
        nv = self.nv
        mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
        try:
            mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        for k, bit in names.items():
            if mask & bit:
                self.reasons.add(k)
        self.samples.append(mhz)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._once()
            except Exception as e:
                self.err = f"{type(e).__name__}: {e}"
                return
            time.sleep(0.005)

    def __enter__(self):
        if self.err is None:
            self._once()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()
            try:
                self._once()
            except Exception:
                pass

    def summary(self):
        if self.err is not None and not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": self.err}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def kv_bytes(ctx: int, heads: int, batch: int) -> int:
    return 2 * batch * ctx * heads * D * 2  # K and V, fp16


# ------------------------------------------------------------------------------------ CPU arm
def use_all_host_cores() -> int:
    """Thread count for the CPU legs.  Must run before torch is imported: a multi-process launcher exports
    OMP_NUM_THREADS=1 to its ranks, which would time the host path on one core."""
    n = os.cpu_count() or 1
    if "torch" not in sys.modules:
        os.environ["OMP_NUM_THREADS"] = str(n)
        os.environ["MKL_NUM_THREADS"] = str(n)
    import torch
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_dense_sample(ctx: int, layers: int, steps: int, warmup: int, budget_s: float):
    """Times the oracle port of the reference's CPU check of dense GQA decode (kind "port": the reference has no
    CPU function of its own for this op; benchmarks/llama_integration_benchmark.py:464-471 is the formula).

    A step is `layers_run` layer passes of ONE sequence, cycling over 4 distinct layer caches (1 GB at 64K: no pass
    finds its input in the host's last-level cache).  `layers_run` is `layers` unless the whole run would exceed
    `budget_s`, in which case every step is a smaller, stated sample.  Returns (dict, layers_run, seconds per step)."""
    cores = use_all_host_cores()
    import torch
    from llm_inference_optimization_b200 import workloads
    from oracle import skv_oracle as oracle

    caches = []
    for i in range(4):
        Q, K, V, scale = workloads.dense_gqa(ctx, seed=1 + i)
        caches.append((Q, K, V))
    oracle.dense_gqa_decode(*caches[0], scale)
    t0 = time.perf_counter()
    oracle.dense_gqa_decode(*caches[1], scale)
    one = time.perf_counter() - t0
    layers_run = layers
    if one * layers * (steps + warmup) > budget_s:
        layers_run = max(1, int(budget_s / ((steps + warmup) * one)))

    def step():
        for l in range(layers_run):
            oracle.dense_gqa_decode(*caches[l % 4], scale)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    per_step = (time.perf_counter() - t0) / steps
    gbs = layers_run * kv_bytes(ctx, HKV, 1) / per_step / 1e9
    sample = (f"{steps} timed steps (after {warmup} warm-up) of {layers_run} layer passes over ONE sequence's fp16 KV "
              f"({ctx} tokens, 8 kv-heads, D=128), fp32 torch restatement of the reference's SDPA+repeat_kv check, "
              f"{cores} threads; {per_step / layers_run * 1e3:.1f} ms per layer pass")
    if layers_run != layers:
        sample += f"; bounded sample: {layers_run} of {layers} layers per step to stay inside {budget_s:.0f} s"
    return {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
            "ms_per_layer": per_step / layers_run * 1e3, "host_cpus": os.cpu_count()}, layers_run, per_step


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    steps, warmup = max(args.steps, 1), max(args.warmup, 0)
    base, layers_run, per_step = cpu_dense_sample(args.ctx, args.layers, steps, warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": per_step * 1e3,
        "us_per_layer": per_step / layers_run * 1e6, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic (seeded N(0,1)/sqrt(D))",
        "config": workload_config(args.ctx, args.layers, world),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "host path: the rate does not depend on N, so at N > 1 rank 0 times one sequence's share of the job",
    }
    print(json.dumps(line), flush=True)


def cpu_other_ops(budget_s: float = 8.0) -> dict:
    """CPU baselines of the other two ops of the path, oracle ports pinned to the reference's own Python functions:
    config 1 (sparse_kv/attention.py:25-38) and config 3 (sparse_kv/eviction.py:30-44)."""
    cores = use_all_host_cores()
    import torch
    from llm_inference_optimization_b200 import workloads
    from oracle import skv_oracle as oracle

    def timed(fn):
        fn()
        t0 = time.perf_counter()
        fn()
        one = time.perf_counter() - t0
        n = max(1, min(50, int(budget_s / max(one, 1e-6))))
        ts = []
        for _ in range(n):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return statistics.median(ts), n

    out = {}
    Q, K, V = workloads.token_sparse_config1()
    sec, n = timed(lambda: oracle.token_sparse_attention(Q, K, V, 256, 4))
    out["config1_token_sparse"] = {"ms": sec * 1e3, "cores": cores, "kind": "port",
                                   "sample": f"median of {n} calls, B=1 H=8 T=1024 D=64 top_k=256 sinks=4, fp32"}
    Ke, Ve, sc = workloads.eviction()
    def ev():
        idx = oracle.eviction_keep_indices(sc, 4096, 64)
        Kw, Vw = oracle.evict_gather(Ke, Ve, idx)
        oracle.quantize_int8(Kw)
        oracle.quantize_int8(Vw)
    sec, n = timed(ev)
    nbytes = eviction_bytes(4, 8, 32768, 128, 4160)
    out["config3_evict_int8"] = {"ms": sec * 1e3, "GBps": nbytes / sec / 1e9, "cores": cores, "kind": "port",
                                 "sample": f"median of {n} calls, B=4 H=8 T=32768 D=128 keep 4096+64, topk+gather+INT8"}
    return out


def eviction_bytes(B, H, T, Dh, keep):
    return B * H * T * 4 + 2 * B * H * keep * Dh * 2 + 2 * B * H * keep * Dh + 2 * B * H * keep * 4 + B * H * keep * 4


# ------------------------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=65536)
    ap.add_argument("--no-extras", action="store_true", help="skip every leg but the headline loop (profiling runs)")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-decode-step", action="store_true", help="skip the full decode-step tokens/s leg")
    ap.add_argument("--no-graph", action="store_true", help="enqueue every launch from Python instead of replaying a CUDA graph of one step")
    args = ap.parse_args()

    if args.impl == "reference":
        reference_arm(args)
        return

    if not args.no_extras and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        use_all_host_cores()   # the CPU baseline legs of this run; before torch is imported
    import torch
    import torch.distributed as dist
    from llm_inference_optimization_b200 import _C, _lib, _workspace

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if HKV % world != 0:
        raise SystemExit(f"cannot partition {HKV} kv-heads over {world} GPUs")
    warmup = max(args.warmup, 3)
    layers = args.layers
    lib = _lib.load()

    # rank-local share of the head-partitioned problem: `world` sequences x (Hkv / world) kv-heads
    hkv_l, hq_l, batch = HKV // world, HQ // world, world
    scale = D ** -0.5

    def make_layers(ctx, n_layers, seed):
        g = torch.Generator(device=dev)
        g.manual_seed(seed + 1000 * rank)
        Ks = [(torch.randn(batch, ctx, hkv_l, D, generator=g, device=dev, dtype=torch.float16) * scale)
              for _ in range(n_layers)]
        Vs = [(torch.randn(batch, ctx, hkv_l, D, generator=g, device=dev, dtype=torch.float16) * scale)
              for _ in range(n_layers)]
        Q = torch.randn(batch, hq_l, D, generator=g, device=dev, dtype=torch.float16) * scale
        return Q, Ks, Vs

    def gather_ranks(x: float) -> list:
        if world == 1:
            return [x]
        t = torch.zeros(world, device=dev, dtype=torch.float64)
        t[rank] = x
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return [float(v) for v in t.tolist()]

    def time_steps(ctx, n_layers, steps, warm, early_kv=False, use_graph=True):
        """ms per step (max over ranks), every rank's ms, and the host's enqueue time per call in us."""
        Q, Ks, Vs = make_layers(ctx, n_layers, seed=1)
        out = torch.empty(batch, hq_l, D, device=dev, dtype=torch.float16)

        def step():
            for l in range(n_layers):
                _C.fused_gqa(Q, Ks[l], Vs[l], scale, out=out)

        # early_kv: the caller's statement that no launch writes the K/V a later launch reads (true here: the
        # caches are static), which lets a launch stream K/V while the previous launch's combine tail drains.
        lib.skv_gqa_set_early_kv(1 if early_kv else 0)
        graph = None
        try:
            for _ in range(warm):
                step()
            torch.cuda.synchronize()
            # the host's enqueue cost per call, from an un-synchronised eager pass (the GPU is still busy when it ends)
            h0 = time.perf_counter()
            step()
            host_us = (time.perf_counter() - h0) * 1e6 / n_layers
            torch.cuda.synchronize()
            if use_graph:
                # One step (32 launches) captured in a CUDA graph and replayed: the timed region then does not depend
                # on how fast each rank's Python loop enqueues (with 8 single-threaded ranks on one host the slowest
                # rank's launch path, not a kernel, set the max-over-ranks time).
                graph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()   # once on the capture stream so that its workspace exists
                torch.cuda.current_stream().wait_stream(side)
                with torch.cuda.graph(graph, stream=side):
                    step()
                run_step = graph.replay
            else:
                run_step = step
            for _ in range(2):
                run_step()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                run_step()
            e1.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
        finally:
            lib.skv_gqa_set_early_kv(0)
            del graph
        ms_all = gather_ranks(e0.elapsed_time(e1) / steps)
        for ws in _workspace.all_of("gqa", dev):
            st = _workspace.status(ws)
            if st != 0:
                raise SystemExit(f"device status word {st}: a bounded wait inside the decode kernel ran out")
        del Ks, Vs
        torch.cuda.empty_cache()
        return max(ms_all), ms_all, max(gather_ranks(host_us))

    sampler = ClockSampler(local)
    with sampler:
        ms_step, ms_ranks, host_us = time_steps(args.ctx, layers, args.steps, warmup, use_graph=not args.no_graph)
    clocks = sampler.summary()

    bytes_layer_rank = kv_bytes(args.ctx, hkv_l, batch)
    us_layer = ms_step * 1e3 / layers
    per_gpu_gbs = bytes_layer_rank / (us_layer * 1e-6) / 1e9
    value = per_gpu_gbs * world
    peak, peak_kind = peaks()
    us_ranks = sorted(m * 1e3 / layers for m in ms_ranks)

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "us_per_layer": us_layer,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic (seeded N(0,1)/sqrt(D), generated on device)",
        "config": workload_config(args.ctx, layers, world),
        "launch": {
            "cuda_graph": not args.no_graph,
            "kv_splits": lib.skv_gqa_decode_splits(batch, args.ctx, hq_l, hkv_l, D, local),
            "order": "default: every launch waits for the one before it (what a real decode step needs, since the "
                     "layer's K/V page is written just before its attention launch); 'early_kv_launches' times the "
                     "opt-in mode for static caches",
        },
        "per_rank_us": {"min": us_ranks[0], "median": us_ranks[len(us_ranks) // 2], "max": us_ranks[-1]},
        "host_us_per_call": host_us,
        "roofline": {
            "bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
            "peak_source": f"{peak_kind} copy bandwidth", "frac_of_nominal_8000": per_gpu_gbs / 8000.0,
            "traffic": NCU_TRAFFIC_BYTES_64K if (args.ctx == 65536 and world == 1) else None,
            "algorithmic_bytes_per_launch": bytes_layer_rank, "avg_launch_us": us_layer,
        },
        "clocks": clocks,
        "gpu_launches": args.steps * layers,
    }

    if not args.no_extras:
        half = max(3, args.steps // 2)
        # ---- the opt-in launch mode for static caches, and the 128K point of the metric (fewer layers: same bytes)
        ms_e, _, _ = time_steps(args.ctx, layers, half, 3, early_kv=True, use_graph=not args.no_graph)
        g_e = bytes_layer_rank / (ms_e * 1e-3 / layers) / 1e9
        line["early_kv_launches"] = {"us_per_layer": ms_e * 1e3 / layers, "gbs_per_gpu": g_e, "frac_of_peak": g_e / peak,
                                     "note": "skv_gqa_set_early_kv(1): a launch streams K/V before the previous launch "
                                             "has completed; valid only while no launch writes K/V (not inside a decode step)"}
        by_ctx = {str(args.ctx): {"us_per_layer": us_layer, "gbs_per_gpu": per_gpu_gbs, "frac_of_peak": per_gpu_gbs / peak}}
        if args.ctx != 131072:
            l128 = max(2, layers // 2)
            ms128, _, _ = time_steps(131072, l128, half, 3, use_graph=not args.no_graph)
            us128 = ms128 * 1e3 / l128
            g128 = kv_bytes(131072, hkv_l, batch) / (us128 * 1e-6) / 1e9
            by_ctx["131072"] = {"us_per_layer": us128, "gbs_per_gpu": g128, "frac_of_peak": g128 / peak}
        line["by_context"] = by_ctx

        # ---- end to end through the public API with HOST buffers
        e2e_steps = max(3, min(args.steps, 10))
        g = torch.Generator().manual_seed(1 + 1000 * rank)
        hQ = (torch.randn(batch, hq_l, D, generator=g) * scale).half().pin_memory()
        hK = torch.empty(batch, args.ctx, hkv_l, D, dtype=torch.float16).pin_memory()
        hV = torch.empty(batch, args.ctx, hkv_l, D, dtype=torch.float16).pin_memory()
        hK.copy_((torch.randn(hK.shape, generator=g) * scale).half())
        hV.copy_((torch.randn(hV.shape, generator=g) * scale).half())
        hO = torch.empty(batch, hq_l, D, dtype=torch.float16).pin_memory()
        dQ, dK, dV = torch.empty_like(hQ, device=dev), torch.empty_like(hK, device=dev), torch.empty_like(hV, device=dev)

        # K and V cross the bus in eight chunks alternating between two copy streams: one stream alone leaves a few
        # percent of the PCIe link unused (51 against 54 GB/s measured)
        c1, c2 = torch.cuda.Stream(), torch.cuda.Stream()
        n_chunks = 8
        # chunks of whole token rows over the flattened (sequence, token) axis: every chunk is one contiguous range of
        # bytes (a slice along the token axis of a [batch, ctx, ...] tensor is not, for batch > 1, and a strided
        # host-to-device copy runs at a seventh of the link rate)
        rows_total = batch * args.ctx
        chunk = (rows_total + n_chunks - 1) // n_chunks
        hKf, hVf, dKf, dVf = (t.view(rows_total, hkv_l, D) for t in (hK, hV, dK, dV))

        def e2e_host_kv():
            cur = torch.cuda.current_stream()
            c1.wait_stream(cur)
            c2.wait_stream(cur)
            for i in range(n_chunks):
                lo, hi = i * chunk, min(rows_total, (i + 1) * chunk)
                with torch.cuda.stream(c1 if i % 2 == 0 else c2):
                    dKf[lo:hi].copy_(hKf[lo:hi], non_blocking=True)
                    dVf[lo:hi].copy_(hVf[lo:hi], non_blocking=True)
            dQ.copy_(hQ, non_blocking=True)
            cur.wait_stream(c1)
            cur.wait_stream(c2)
            o = _C.fused_gqa(dQ, dK, dV, scale)
            hO.copy_(o, non_blocking=True)

        def e2e_resident():
            dQ.copy_(hQ, non_blocking=True)
            o = _C.fused_gqa(dQ, dK, dV, scale)
            hO.copy_(o, non_blocking=True)

        def timed(fn, n):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return max(gather_ranks(e0.elapsed_time(e1) / n))

        ms_e2e = timed(e2e_host_kv, e2e_steps)
        ms_res = timed(e2e_resident, e2e_steps * 20)
        qo = hQ.numel() * 2
        line["e2e"] = {
            "value": world * bytes_layer_rank / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": qo + bytes_layer_rank, "d2h_bytes_per_step": qo,
            "ms_per_layer": ms_e2e, "steps": e2e_steps,
            "note": "one layer per step: pinned host Q, K, V -> device, fused_gqa(), output -> pinned host; PCIe-bound by "
                    "construction (the whole KV cache crosses the bus every step); every rank has its own link",
        }
        line["e2e_resident_kv"] = {
            "value": world * bytes_layer_rank / (ms_res * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": qo, "d2h_bytes_per_step": qo, "ms_per_layer": ms_res,
            "note": "the reference API takes CUDA-resident caches (gqa_decode.cu:225): only the query goes in "
                    "and the output comes back each step",
        }
        del dK, dV, hK, hV, dKf, dVf, hKf, hVf

        # ---- the other two ops of the path at their configs, head-partitioned like the headline (weak scaling)
        line["other_configs"] = other_configs(dev, world, rank, peak, gather_ranks)

        # ---- CPU baselines next to it (rank 0, single-GPU run only)
        if world == 1 and rank == 0:
            base, _, _ = cpu_dense_sample(args.ctx, layers, 3, 1, budget_s=15.0)
            line["cpu_baseline"] = base
            line["cpu_baseline_other_ops"] = cpu_other_ops()
            line["reference_cuda"] = reference_cuda_leg(dev)

    if not args.no_extras and not args.no_decode_step:
        # ---- the other half of the metric: tokens/s of the full tensor-parallel decode step (all ranks take part)
        from llm_inference_optimization_b200 import bench_decode
        torch.cuda.empty_cache()
        try:
            res = bench_decode.run(steps=10, warmup=3, hybrid_dense_layers=16, mixed_pages=True)
        except Exception as e:  # reported, never fatal for the headline line
            res = {"error": f"{type(e).__name__}: {e}"}
        if rank == 0:
            line["decode_step"] = res

    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def other_configs(dev, world, rank, peak, gather_ranks) -> dict:
    """Fused eviction + INT8 (config 3) and Quest block-sparse decode over paged FP8 (config 4) on every rank's share:
    rank r owns H / world heads of world x the batch, so the work per GPU is the configuration's own."""
    import torch
    from llm_inference_optimization_b200 import eviction, paged

    flush = torch.zeros(64 << 20, dtype=torch.int32, device=dev)   # 256 MB read between calls: larger than L2

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.max()
            flush.max()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return max(gather_ranks(statistics.median(ts)))

    out = {}
    g = torch.Generator(device=dev)
    g.manual_seed(77 + rank)
    # config 3
    B, H, T, Dh, budget, recent = 4 * world, 8 // world, 32768, 128, 4096, 64
    K = torch.randn((B, H, T, Dh), device=dev, generator=g, dtype=torch.float32).half()
    V = torch.randn((B, H, T, Dh), device=dev, generator=g, dtype=torch.float32).half()
    sc = torch.rand((B, H, T), device=dev, generator=g, dtype=torch.float32)
    us = timed(lambda: eviction.fused_kv_evict(K, V, sc, budget, recent_tokens=recent, quant="int8", return_aux=True))
    nbytes = eviction_bytes(B, H, T, Dh, budget + recent)
    out["config3_evict_int8"] = {"us": us, "GBps_total": world * nbytes / us / 1e3, "frac_of_peak_per_gpu": nbytes / us / 1e3 / peak,
                                 "algorithmic_MB_per_gpu": nbytes / 1e6, "per_gpu_shape": [B, H, T, Dh]}
    del K, V, sc
    # config 4
    B, Hq, Hkv, T, P, bs, k = 8 * world, 32 // world, 8 // world, 131072, 16, 64, 8
    pages = B * T // P
    buf = torch.randint(0, 256, (pages, Hkv, paged.RECORD_ROWS, 128), device=dev, generator=g, dtype=torch.uint8)
    buf[:, :, :32] = torch.where((buf[:, :, :32] & 0x7F) == 0x7F, buf[:, :, :32] & 0xFE, buf[:, :, :32])  # no NaN codes
    table = torch.randperm(pages, device=dev, generator=g).to(torch.int32).view(B, T // P)
    kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table, None, B)
    kv.k_scale.copy_(torch.rand(kv.k_scale.shape, device=dev, generator=g) * 0.01 + 0.005)
    kv.v_scale.copy_(torch.rand(kv.v_scale.shape, device=dev, generator=g) * 0.01 + 0.005)
    Q = torch.randn((B, Hq, Dh), device=dev, generator=g, dtype=torch.float32).half()
    meta = paged.build_block_meta(kv, bs)
    us = timed(lambda: paged.quest_sparse_decode(Q, kv, meta, Dh ** -0.5, bs, k))
    nbytes = B * Hkv * (T // bs) * 2 * Dh * 2 + B * Hq * k * bs * 2 * (Dh + 4) + B * Hq * k * (bs // P) * 4
    out["config4_quest_fp8"] = {"us": us, "GBps_total": world * nbytes / us / 1e3, "frac_of_peak_per_gpu": nbytes / us / 1e3 / peak,
                                "algorithmic_MB_per_gpu": nbytes / 1e6, "per_gpu_shape": {"B": B, "Hq": Hq, "Hkv": Hkv, "ctx": T}}
    del buf, kv, meta, flush
    torch.cuda.empty_cache()
    return out


def reference_cuda_leg(dev) -> dict:
    """The reference's OWN CUDA kernels (its three .cu files compiled unchanged for sm_100a, oracle/build_ref.py) timed
    on this GPU beside this library's kernels, at the shapes of the reference's sweep (benchmarks/run_benchmarks.py:22-80:
    B=1, H=32, D=128; the dense kernel with 8 kv-heads).  Checker-side code: nothing in the product path loads it."""
    import torch
    from llm_inference_optimization_b200 import _C
    from oracle import build_ref
    if not build_ref.available():
        return {"unavailable": "oracle/_ref holds no built module (run `python oracle/build_ref.py` where the reference checkout is)"}
    ref = build_ref.load()

    def t(fn, it):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(it):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / it * 1e3

    res = {}
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    for N in (4096, 16384, 65536):
        Q = (torch.randn(1, 32, 128, device=dev, generator=g) * 128 ** -0.5).half()
        K = (torch.randn(1, N, 8, 128, device=dev, generator=g) * 128 ** -0.5).half()
        V = (torch.randn(1, N, 8, 128, device=dev, generator=g) * 128 ** -0.5).half()
        Q4 = torch.randn(1, 32, 1, 128, device=dev, generator=g).half()
        K4 = torch.randn(1, 32, N, 128, device=dev, generator=g).half()
        V4 = torch.randn(1, 32, N, 128, device=dev, generator=g).half()
        res[str(N)] = {
            "fused_gqa_us": {"reference": t(lambda: ref.fused_gqa(Q, K, V, 128 ** -0.5), 3),
                             "ours": t(lambda: _C.fused_gqa(Q, K, V, 128 ** -0.5), 20)},
            "kv_evict_quant_forward_top32_us": {"reference": t(lambda: ref.kv_evict_quant_forward(Q4, K4, V4, 32, False), 3),
                                                "ours": t(lambda: _C.kv_evict_quant_forward(Q4, K4, V4, 32, False), 20)},
            "sparse_attention_forward_64x8_us": {"reference": t(lambda: ref.sparse_attention_forward(Q4, K4, V4, 64, 8), 3),
                                                 "ours": t(lambda: _C.sparse_attention_forward(Q4, K4, V4, 64, 8), 20)},
        }
        del K, V, K4, V4
    res["note"] = ("back-to-back calls on one input (L2-warm at 4K and 16K for both sides); the reference's token kernel "
                   "keeps an approximate top-k, ours is exact")
    return res


if __name__ == "__main__":
    main()
