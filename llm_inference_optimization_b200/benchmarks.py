"""Kernel-level sweep of the decode path on one B200: the counterpart of the reference's
``benchmarks/run_benchmarks.py`` (its 4K-128K sweep at B=1, H=32, D=128, :22-80) for the kernels here.

    python -m llm_inference_optimization_b200.benchmarks [--only dense,paged,token,block,evict,quest] [--iters 20]

Prints one JSON line per (workload, size): median CUDA-event time of the whole operator (all of its
launches), the algorithmic bytes, GB/s and the fraction of the measured HBM copy bandwidth.  Inputs are
generated on the device (seeded); before every timed call a 512 MB buffer is READ, which replaces the L2
contents with clean lines (a written buffer would leave dirty lines whose write-back competes with the call).
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
import sys
from pathlib import Path

import torch

from . import _C, eviction, paged

ROOT = Path(__file__).resolve().parents[1]


def hbm_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class Timer:
    last_mean = None   # mean of the most recent measurement, picked up (and cleared) by emit()

    def __init__(self, dev, iters):
        self.dev, self.iters = dev, iters
        self.flush_buf = torch.zeros(128 << 20, dtype=torch.int32, device=dev)

    def __call__(self, fn, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize(self.dev)
        times = []
        for _ in range(self.iters):
            for _ in range(3):  # read-only passes over 512 MB: evict the previous call's data, leave L2 clean, and
                self.flush_buf.max()  # keep the GPU busy long enough for the host to enqueue the whole timed call
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(self.dev)
            times.append(e0.elapsed_time(e1) * 1e3)
        # CUDA event pairs around one short call resolve about 2 us here (the medians of the short ops land on a
        # 2.05 us grid); the mean over the iterations is kept beside the median for telling such ops apart
        Timer.last_mean = statistics.fmean(times)
        return statistics.median(times), min(times)


def emit(name, cfg, us, us_min, nbytes, peak, peak_kind, **extra):
    gbs = nbytes / us / 1e3
    if Timer.last_mean is not None:
        extra = {"us_mean": round(Timer.last_mean, 2), **extra}
        Timer.last_mean = None
    line = {"workload": name, **cfg, "us": round(us, 2), "us_min": round(us_min, 2), "algorithmic_MB": round(nbytes / 1e6, 2),
            "GBps": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3), "peak_GBps": peak, "peak_source": peak_kind, **extra}
    print(json.dumps(line), flush=True)
    RESULTS.append(line)


RESULTS: list = []   # every line printed in this process, for the --csv / --json files


def randn16(shape, dev, g, scale=1.0):
    return (torch.randn(shape, device=dev, generator=g, dtype=torch.float32) * scale).half()


def random_pools(num_pages, Hkv, P, D, dev, g, fp8=True):
    codes = torch.randint(0, 256, (num_pages, Hkv, P, D), device=dev, generator=g, dtype=torch.uint8)
    if fp8:
        codes = torch.where((codes & 0x7F) == 0x7F, codes & 0xFE, codes)  # no NaN patterns
        codes = codes.view(torch.float8_e4m3fn)
    else:
        codes = codes.view(torch.int8)
    scales = torch.rand((num_pages, Hkv, P), device=dev, generator=g, dtype=torch.float32) * 0.01 + 0.005
    return codes, scales


def bench_dense(t, dev, g, peak, pk):
    D, Hq, Hkv = 128, 32, 8
    for N in (4096, 16384, 65536, 131072):
        Q = randn16((1, Hq, D), dev, g, D ** -0.5)
        K = randn16((1, N, Hkv, D), dev, g, D ** -0.5)
        V = randn16((1, N, Hkv, D), dev, g, D ** -0.5)
        out = torch.empty_like(Q)
        us, mn = t(lambda: _C.fused_gqa(Q, K, V, D ** -0.5, out=out))
        emit("dense_gqa_f16", {"B": 1, "Hq": Hq, "Hkv": Hkv, "D": D, "ctx": N}, us, mn, 2 * N * Hkv * D * 2, peak, pk)
        del K, V


def bench_paged(t, dev, g, peak, pk):
    D, Hq, Hkv, P = 128, 32, 8, 16
    for fp8 in (True, False):
        for B, N in ((1, 65536), (1, 131072), (16, 65536)):
            pages = B * N // P
            kp, ks = random_pools(pages, Hkv, P, D, dev, g, fp8)
            vp, vs = random_pools(pages, Hkv, P, D, dev, g, fp8)
            table = torch.randperm(pages, device=dev, generator=g).to(torch.int32).view(B, N // P)
            Q = randn16((B, Hq, D), dev, g)
            out = torch.empty_like(Q)
            us, mn = t(lambda: _C.fused_gqa_paged(Q, kp, vp, ks, vs, table, None, D ** -0.5, out=out))
            nbytes = 2 * B * N * Hkv * (D + 4)
            emit("dense_gqa_paged_" + ("fp8" if fp8 else "int8"), {"B": B, "Hq": Hq, "Hkv": Hkv, "D": D, "ctx": N, "page": P,
                                                                    "layout": "separate pools"}, us, mn, nbytes, peak, pk)
            buf = paged.pack_fused(kp, vp, ks, vs)
            del kp, vp, ks, vs
            kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn if fp8 else torch.int8, table, None, B)
            us, mn = t(lambda: _C.fused_gqa_paged(Q, kv.k_pool, kv.v_pool, kv.k_scale, kv.v_scale, table, None, D ** -0.5, out=out))
            emit("dense_gqa_paged_" + ("fp8" if fp8 else "int8"), {"B": B, "Hq": Hq, "Hkv": Hkv, "D": D, "ctx": N, "page": P,
                                                                    "layout": "fused page records"}, us, mn, nbytes, peak, pk)
            del buf, kv


def bench_mixed(t, dev, g, peak, pk):
    """Dense decode over mixed-precision page records (8-bit K, 4-bit V): 200 bytes per token and head against the
    264 of an all-8-bit cache.  Random codes with fixed scales."""
    D, Hq, Hkv, P = 128, 32, 8, 16
    for fp8 in (True, False):
        for B, N in ((1, 65536), (1, 131072), (16, 65536)):
            pages = B * N // P
            buf = torch.randint(0, 256, (pages, Hkv, paged.MIXED_RECORD_ROWS, 128), device=dev, generator=g, dtype=torch.uint8)
            if fp8:   # no NaN codes among the keys
                buf[:, :, :16] = torch.where((buf[:, :, :16] & 0x7F) == 0x7F, buf[:, :, :16] & 0xFE, buf[:, :, :16])
            table = torch.randperm(pages, device=dev, generator=g).to(torch.int32).view(B, N // P)
            kv = paged.PagedKV.from_mixed(buf, torch.float8_e4m3fn if fp8 else torch.int8, table, None, B)
            kv.k_scale.fill_(0.008)
            kv.v_scale.fill_(0.05)
            Q = randn16((B, Hq, D), dev, g)
            out = torch.empty_like(Q)
            us, mn = t(lambda: kv.decode(Q, D ** -0.5, out=out))
            nbytes = B * N * Hkv * (D + D // 2 + 8)
            emit("dense_gqa_paged_" + ("fp8" if fp8 else "int8") + "_k_int4_v", {"B": B, "Hq": Hq, "Hkv": Hkv, "D": D, "ctx": N, "page": P,
                                                                                  "layout": "mixed-precision page records"},
                 us, mn, nbytes, peak, pk, us_per_8bit_byte_count=round(us * 264 / 200, 2))
            del buf, kv


def bench_paged_stream(t, dev, g, peak, pk):
    """One sequence over a paged FP8 cache the way a model runs it: launches back to back over eight layers' caches
    (1.1 GB per cycle at 64K, so no launch finds its input in L2), CUDA events around 25 cycles.  The isolated-call
    figures of `paged` carry the launch, ramp and last-combine tail of a single launch, which consecutive launches
    overlap (programmatic dependent launch)."""
    D, Hq, Hkv, P, L = 128, 32, 8, 16, 8
    for N in (65536, 131072):
        pages = N // P
        caches = []
        for _ in range(L):
            buf = torch.randint(0, 256, (pages, Hkv, paged.RECORD_ROWS, 128), device=dev, generator=g, dtype=torch.uint8)
            buf[:, :, :32] = torch.where((buf[:, :, :32] & 0x7F) == 0x7F, buf[:, :, :32] & 0xFE, buf[:, :, :32])
            kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, None, None, 1)
            kv.k_scale.fill_(0.008)
            kv.v_scale.fill_(0.008)
            caches.append(kv)
        table = torch.randperm(pages, device=dev, generator=g).to(torch.int32).view(1, pages)
        Q = randn16((1, Hq, D), dev, g)
        out = torch.empty_like(Q)

        def cycle():
            for kv in caches:
                _C.fused_gqa_paged(Q, kv.k_pool, kv.v_pool, kv.k_scale, kv.v_scale, table, None, D ** -0.5, out=out)

        for _ in range(3):
            cycle()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 25
        e0.record()
        for _ in range(reps):
            cycle()
        e1.record()
        torch.cuda.synchronize(dev)
        us = e0.elapsed_time(e1) * 1e3 / (reps * L)
        emit("dense_gqa_paged_fp8_back_to_back", {"B": 1, "Hq": Hq, "Hkv": Hkv, "D": D, "ctx": N, "page": P,
                                                   "layout": "fused page records", "layers_per_cycle": L},
             us, us, 2 * N * Hkv * (D + 4), peak, pk)
        del caches


def bench_ragged(t, dev, g, peak, pk):
    """The decode step's attention launch: batch 16, context lengths uniform in 8K..128K (the seed of bench_decode), FP8
    fused page records, with the kv-heads one rank owns at tensor-parallel degree 8 (one) and 1 (eight)."""
    from . import _lib
    lib = _lib.load()
    D, P, B = 128, 16, 16
    lens = torch.randint(8192, 131073, (B,), generator=torch.Generator().manual_seed(4), dtype=torch.int32)
    cap = (int(lens.max()) + 15) // 16
    pages_per_seq = [(int(n) + 15) // 16 for n in lens.tolist()]
    total = sum(pages_per_seq)
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(4))
    table = torch.zeros((B, cap), dtype=torch.int32)
    o = 0
    for b, n in enumerate(pages_per_seq):
        table[b, :n] = perm[o:o + n].to(torch.int32)
        o += n
    table, dl = table.to(dev), lens.to(dev)
    for Hkv in (1, 2, 4, 8):
        Hq = 4 * Hkv
        buf = torch.randint(0, 256, (total, Hkv, paged.RECORD_ROWS, 128), device=dev, generator=g, dtype=torch.uint8)
        buf[:, :, :32] = torch.where((buf[:, :, :32] & 0x7F) == 0x7F, buf[:, :, :32] & 0xFE, buf[:, :, :32])
        kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table, dl, B)
        kv.k_scale.copy_(torch.rand(kv.k_scale.shape, device=dev, generator=g) * 0.004 + 0.006)
        kv.v_scale.copy_(torch.rand(kv.v_scale.shape, device=dev, generator=g) * 0.004 + 0.006)
        Q = randn16((B, Hq, D), dev, g)
        out = torch.empty_like(Q)
        nbytes = int(lens.sum()) * Hkv * 2 * (D + 4)
        for worklist in (1, 2, 3, 0):
            lib.skv_gqa_set_ragged_worklist(worklist)
            try:
                us, mn = t(lambda: _C.fused_gqa_paged(Q, kv.k_pool, kv.v_pool, kv.k_scale, kv.v_scale, table, dl, D ** -0.5,
                                                      max_seq_len=cap * 16, out=out))
            finally:
                lib.skv_gqa_set_ragged_worklist(1)
            emit("dense_gqa_paged_fp8_ragged", {"B": B, "Hq": Hq, "Hkv": Hkv, "D": D, "ctx": "8K..128K (sum %d)" % int(lens.sum()),
                                                 "schedule": f"work list from the real lengths, {worklist} wave(s)" if worklist else "static split plan"},
                 us, mn, nbytes, peak, pk)
        del buf, kv



def bench_token(t, dev, g, peak, pk):
    D, H = 128, 32
    for T in (4096, 16384, 65536, 131072):
        Q, K, V = randn16((1, H, 1, D), dev, g), randn16((1, H, T, D), dev, g), randn16((1, H, T, D), dev, g)
        us, mn = t(lambda: _C.token_sparse_decode(Q, K, V, 32, 4))
        emit("token_sparse_top32", {"B": 1, "H": H, "D": D, "ctx": T, "top_k": 32, "sink": 4}, us, mn,
             H * T * D * 2 + H * T * 4 + 36 * H * D * 2, peak, pk)
        del K, V


def bench_block(t, dev, g, peak, pk):
    D, H = 128, 32
    for T in (4096, 16384, 65536, 131072):
        Q, K, V = randn16((1, H, 1, D), dev, g), randn16((1, H, T, D), dev, g), randn16((1, H, T, D), dev, g)
        us, mn = t(lambda: _C.sparse_attention_forward(Q, K, V, 64, 8))
        emit("block_sparse_mean_64x8", {"B": 1, "H": H, "D": D, "ctx": T, "block": 64, "top_k_blocks": 8}, us, mn,
             H * T * D * 2 + H * 512 * D * 2, peak, pk)
        del K, V


def bench_evict(t, dev, g, peak, pk):
    B, H, T, D, budget, recent = 4, 8, 32768, 128, 4096, 64
    K, V = randn16((B, H, T, D), dev, g), randn16((B, H, T, D), dev, g)
    scores = torch.rand((B, H, T), device=dev, generator=g, dtype=torch.float32)
    keep = budget + recent
    from . import _lib
    lib = _lib.load()
    nbytes = B * H * T * 4 + 2 * B * H * keep * D * 2 + 2 * B * H * keep * D + 2 * B * H * keep * 4 + B * H * keep * 4
    for quant in ("int8", "fp8"):
        for fused in (1, 0):
            lib.skv_kv_evict_set_fused(fused)
            try:
                us, mn = t(lambda: eviction.fused_kv_evict(K, V, scores, budget, recent_tokens=recent, quant=quant, return_aux=True))
            finally:
                lib.skv_kv_evict_set_fused(0)
            emit("kv_evict_quant_" + quant, {"B": B, "H": H, "T": T, "D": D, "budget": budget, "recent": recent,
                                             "launches": "one (cluster selects and gathers)" if fused else "two (select, gather)"},
                 us, mn, nbytes, peak, pk)


def bench_quest(t, dev, g, peak, pk):
    B, Hq, Hkv, D, T, P, bs, k = 8, 32, 8, 128, 131072, 16, 64, 8
    pages = B * T // P
    kp, ks = random_pools(pages, Hkv, P, D, dev, g, True)
    vp, vs = random_pools(pages, Hkv, P, D, dev, g, True)
    table = torch.randperm(pages, device=dev, generator=g).to(torch.int32).view(B, T // P)
    kv = paged.PagedKV(kp, vp, ks, vs, table, None, B)
    Q = randn16((B, Hq, D), dev, g)
    us, mn = t(lambda: paged.build_block_meta(kv, bs))
    emit("quest_build_meta_fp8", {"B": B, "Hkv": Hkv, "D": D, "ctx": T, "block": bs}, us, mn,
         B * Hkv * T * (D + 4) + B * Hkv * (T // bs) * 2 * D * 2, peak, pk)
    meta = paged.build_block_meta(kv, bs)
    us, mn = t(lambda: paged.quest_sparse_decode(Q, kv, meta, D ** -0.5, bs, k))
    nbytes = B * Hkv * (T // bs) * 2 * D * 2 + B * Hq * k * bs * 2 * (D + 4) + B * Hq * k * (bs // P) * 4
    emit("quest_sparse_decode_fp8", {"B": B, "Hq": Hq, "Hkv": Hkv, "D": D, "ctx": T, "page": P, "block": bs, "top_k_blocks": k},
         us, mn, nbytes, peak, pk)


ALL = {"dense": bench_dense, "paged": bench_paged, "mixed": bench_mixed, "paged_stream": bench_paged_stream, "ragged": bench_ragged, "token": bench_token, "block": bench_block, "evict": bench_evict,
       "quest": bench_quest}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=",".join(ALL))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--csv", help="also write the results as a CSV table (the reference's sweep writes CSV and JSON, "
                                  "benchmarks/run_benchmarks.py:64-80)")
    ap.add_argument("--json", help="also write the results as one JSON array")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: there is no CPU fallback")
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    peak, pk = hbm_peak()
    t = Timer(dev, args.iters)
    for name in args.only.split(","):
        ALL[name.strip()](t, dev, g, peak, pk)
        torch.cuda.empty_cache()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(RESULTS, f, indent=1)
    if args.csv:
        import csv
        cols = []
        for r in RESULTS:
            cols += [k for k in r if k not in cols]
        with open(args.csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=cols)
            w.writeheader()
            w.writerows(RESULTS)


if __name__ == "__main__":
    main(sys.argv[1:])
