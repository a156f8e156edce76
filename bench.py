#!/usr/bin/env python
"""Benchmark of the dense GQA decode-attention hot path (the metric the baseline is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--ctx 65536]

Workload ("config 2", Llama-3.1-8B layer shape): B=1 per GPU-share, Hq=32, Hkv=8, D=128, fp16 KV
cache of `ctx` tokens in the reference's [B, N, Hkv, D] layout, one query token.  One STEP is one
decode pass over the attention of a 32-layer model: 32 launches of the decode kernel, each over
its own layer's KV cache (32 x 268 MB at 64K, so consecutive launches never find their input in
the 126 MB L2).  `value` is KV bytes streamed per second (GB/s) with the caches resident in HBM;
`us_per_layer` is the same time divided by 32.

With N > 1 GPUs the path is partitioned by KV head and needs no collective: rank r owns
Hkv / N kv-heads (and their 4 query heads each) of N sequences, so the work per GPU stays that
of one sequence ("weak" scaling) while the global batch grows with N.

`--impl reference` times the CPU restatement of the reference's own check of this path
(fp32 softmax(QK^T)V over repeat_kv-expanded heads) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = 32
HQ, HKV, D = 32, 8, 128
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per launch of the decode kernel at 64K measured with ncu (dram__bytes_read.sum +
# dram__bytes_write.sum, see profiles/); None until a capture has been summarised there.
NCU_TRAFFIC_BYTES_64K = 272_600_000  # profiles/gqa_decode_f16_ctx65536.md


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


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
def cpu_reference_run(ctx: int, steps: int, warmup: int, budget_s: float = 20.0):
    """Times the oracle port of the reference's CPU check of dense GQA decode on one layer."""
    import torch
    from llm_inference_optimization_b200 import workloads
    from oracle import skv_oracle as oracle

    Q, K, V, scale = workloads.dense_gqa(ctx)
    for _ in range(max(1, min(warmup, 3))):
        oracle.dense_gqa_decode(Q, K, V, scale)
    t0 = time.perf_counter()
    oracle.dense_gqa_decode(Q, K, V, scale)
    one = time.perf_counter() - t0
    reps = max(1, min(steps, int(budget_s / max(one, 1e-6))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.dense_gqa_decode(Q, K, V, scale)
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    gbs = kv_bytes(ctx, HKV, 1) / med / 1e9
    return {
        "value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"{reps} passes over ONE layer's fp16 KV ({ctx} tokens, 8 kv-heads, D=128) with the fp32 torch "
                  f"restatement of the reference's SDPA+repeat_kv check; median {med * 1e3:.1f} ms/layer",
        "ms_per_layer": med * 1e3, "host_cpus": os.cpu_count(),
    }, reps, med


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, reps, med = cpu_reference_run(args.ctx, max(args.steps, 1), args.warmup)
    line = {
        "impl": "reference", "metric": "decode_attn_kv_stream_bandwidth", "value": base["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": reps, "warmup": min(args.warmup, 3), "ms_per_step": med * 1e3 * LAYERS,
        "us_per_layer": med * 1e6, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 storage, f32 accumulate", "data": "synthetic (seeded N(0,1)/sqrt(D))",
        "config": {"workload": f"config2 dense GQA decode, Llama-3.1-8B layer shape, context {args.ctx}",
                   "B": 1, "Hq": HQ, "Hkv": HKV, "D": D, "ctx": args.ctx,
                   "note": "a step of this arm is ONE layer (bounded sample); ms_per_step is scaled to 32 layers"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=65536)
    ap.add_argument("--no-extras", action="store_true", help="skip the 128K / e2e / CPU legs (profiling runs)")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-decode-step", action="store_true", help="skip the full decode-step tokens/s leg")
    args = ap.parse_args()

    if args.impl == "reference":
        reference_arm(args)
        return

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

    def time_steps(ctx, n_layers, steps, warm, early_kv=True):
        Q, Ks, Vs = make_layers(ctx, n_layers, seed=1)
        out = torch.empty(batch, hq_l, D, device=dev, dtype=torch.float16)
        # The layers' caches are static during the timed region, so a launch may stream K/V while the previous
        # launch's combine tail drains; with early_kv off every launch first waits for the one before.
        _lib.load().skv_gqa_set_early_kv(1 if early_kv else 0)

        def step():
            for l in range(n_layers):
                _C.fused_gqa(Q, Ks[l], Vs[l], scale, out=out)

        for _ in range(warm):
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
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        _lib.load().skv_gqa_set_early_kv(0)
        st = _workspace.status(_workspace.get("gqa", 0, dev))
        if st != 0:
            raise SystemExit(f"device status word {st}: a bounded wait inside the decode kernel ran out")
        del Ks, Vs
        torch.cuda.empty_cache()
        return ms / steps

    sampler = ClockSampler(local)
    with sampler:
        ms_step = time_steps(args.ctx, layers, args.steps, warmup)
    clocks = sampler.summary()

    bytes_layer_rank = kv_bytes(args.ctx, hkv_l, batch)
    us_layer = ms_step * 1e3 / layers
    per_gpu_gbs = bytes_layer_rank / (us_layer * 1e-6) / 1e9
    value = per_gpu_gbs * world
    peak, peak_kind = peaks()

    line = {
        "metric": "decode_attn_kv_stream_bandwidth", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "us_per_layer": us_layer,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 storage, f32 accumulate", "data": "synthetic (seeded N(0,1)/sqrt(D), generated on device)",
        "config": {
            "workload": f"config2 dense GQA decode, Llama-3.1-8B layer shape, context {args.ctx}, "
                        f"{layers} layers per step",
            "global_batch": batch, "Hq": HQ, "Hkv": HKV, "D": D, "ctx": args.ctx, "layers_per_step": layers,
            "partition": f"kv-head: {hkv_l} kv-heads x {batch} sequences per GPU, no collective",
            "l2": f"each launch reads its own layer's {bytes_layer_rank / 1e6:.0f} MB cache; "
                  f"{layers * bytes_layer_rank / 1e9:.1f} GB cycle >> 126 MB L2",
            "kv_splits": _lib.load().skv_gqa_decode_splits(batch, args.ctx, hq_l, hkv_l, D, local),
            "launch_order": "skv_gqa_set_early_kv(1): the caches are static while timed, so a launch streams K/V "
                            "before the previous launch has completed (q, out, workspace stay ordered); the "
                            "default fully ordered launches are timed in 'ordered_launches'",
        },
        "roofline": {
            "bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
            "peak_source": f"{peak_kind} copy bandwidth", "frac_of_nominal_8000": per_gpu_gbs / 8000.0,
            "traffic": NCU_TRAFFIC_BYTES_64K if args.ctx == 65536 else None,
            "algorithmic_bytes_per_launch": bytes_layer_rank, "avg_launch_us": us_layer,
        },
        "clocks": clocks,
        "gpu_launches": args.steps * layers,
    }

    if not args.no_extras:
        # ---- 128K point of the metric (fewer layers: same bytes per step)
        if args.ctx != 131072:
            l128 = max(2, layers // 2)
            ms128 = time_steps(131072, l128, max(3, args.steps // 2), 3)
            us128 = ms128 * 1e3 / l128
            g128 = kv_bytes(131072, hkv_l, batch) / (us128 * 1e-6) / 1e9
            ms_ord = time_steps(args.ctx, layers, max(3, args.steps // 2), 3, early_kv=False)
            g_ord = kv_bytes(args.ctx, hkv_l, batch) / (ms_ord * 1e-3 / layers) / 1e9
            line["ordered_launches"] = {"us_per_layer": ms_ord * 1e3 / layers, "gbs_per_gpu": g_ord,
                                        "frac_of_peak": g_ord / peak,
                                        "note": "default launch order: every launch waits for the one before"}
            line["by_context"] = {
                str(args.ctx): {"us_per_layer": us_layer, "gbs_per_gpu": per_gpu_gbs, "frac_of_peak": per_gpu_gbs / peak},
                "131072": {"us_per_layer": us128, "gbs_per_gpu": g128, "frac_of_peak": g128 / peak},
            }

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

        def e2e_host_kv():
            dQ.copy_(hQ, non_blocking=True)
            dK.copy_(hK, non_blocking=True)
            dV.copy_(hV, non_blocking=True)
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
            ms = e0.elapsed_time(e1) / n
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

        ms_e2e = timed(e2e_host_kv, e2e_steps)
        ms_res = timed(e2e_resident, e2e_steps * 20)
        qo = hQ.numel() * 2
        line["e2e"] = {
            "value": world * bytes_layer_rank / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": qo + bytes_layer_rank, "d2h_bytes_per_step": qo,
            "ms_per_layer": ms_e2e, "steps": e2e_steps,
            "note": "one layer per step: pinned host Q, K, V -> device, fused_gqa(), output -> pinned host; "
                    "PCIe-bound because the whole KV cache crosses the bus every step",
        }
        line["e2e_resident_kv"] = {
            "value": world * bytes_layer_rank / (ms_res * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": qo, "d2h_bytes_per_step": qo, "ms_per_layer": ms_res,
            "note": "the reference API takes CUDA-resident caches (gqa_decode.cu:225): only the query goes in "
                    "and the output comes back each step",
        }
        del dK, dV, hK, hV

        # ---- CPU baseline next to it (rank 0, single-GPU run only)
        if world == 1 and rank == 0:
            base, _, _ = cpu_reference_run(args.ctx, 1000, 2, budget_s=15.0)
            line["cpu_baseline"] = base

    if not args.no_extras and not args.no_decode_step:
        # ---- the other half of the metric: tokens/s of the full tensor-parallel decode step (all ranks take part)
        from llm_inference_optimization_b200 import bench_decode
        torch.cuda.empty_cache()
        try:
            res = bench_decode.run(steps=10, warmup=3)
        except Exception as e:  # reported, never fatal for the headline line
            res = {"error": f"{type(e).__name__}: {e}"}
        if rank == 0:
            line["decode_step"] = res

    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
