"""The range-checking debug library (the same kernels compiled with -DSKV_BOUNDS) runs the hot path clean.

compute-sanitizer is not available where these kernels are tested, so the debug build checks itself: every
data-dependent index goes through a range check that records the first violation and clamps the index, and the
driver below additionally surrounds caller-provided outputs with canary bytes.  The library is chosen per process
(SKV_B200_LIB), so the driver runs in a child process; it prints one JSON line.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu

DRIVER = r'''
import ctypes as C, json, sys
import torch
sys.path.insert(0, %(root)r)
from llm_inference_optimization_b200 import _C, _lib, eviction, paged, workloads
from oracle import skv_oracle as oracle
lib = _lib.load()
dev = torch.device("cuda", 0)
res = {"lib": str(_lib.LIB_PATH)}

def word(name):
    f = getattr(lib, name); f.restype = C.c_int; f.argtypes = [C.POINTER(C.c_int)]
    v = C.c_int(-1); assert f(C.byref(v)) == 0
    return v.value

# the instrumentation itself: an in-range index passes, an out-of-range one is clamped to 0 and its line recorded
lib.skv_debug_bounds_selftest.restype = C.c_int
lib.skv_debug_bounds_selftest.argtypes = [C.POINTER(C.c_int)] * 3
a, b, c = C.c_int(-1), C.c_int(-1), C.c_int(-1)
assert lib.skv_debug_bounds_selftest(C.byref(a), C.byref(b), C.byref(c)) == 0
res["selftest"] = [a.value, b.value, c.value > 0]

def canary(shape, dtype):
    """A tensor of `shape` in the middle of a larger buffer filled with 0xA5 bytes."""
    n = int(torch.tensor(shape).prod()) * torch.empty((), dtype=dtype).element_size()
    raw = torch.full((n + 8192,), 0xA5, dtype=torch.uint8, device=dev)
    return raw, raw[4096:4096 + n].view(dtype).view(shape)

def intact(raw):
    return bool((raw[:4096] == 0xA5).all() and (raw[-4096:] == 0xA5).all())

ok = {}
# dense fp16 decode, ragged length, caller-provided output between canaries
Q, K, V, scale = workloads.dense_gqa(5000, B=2)
lens = torch.tensor([5000, 77], dtype=torch.int32, device=dev)
raw, out = canary((2, 32, 128), torch.float16)
_C.fused_gqa(Q.to(dev), K.to(dev), V.to(dev), scale, seq_lens=lens, out=out)
want = oracle.dense_gqa_decode(Q, K, V, scale, lens.cpu())
ok["dense"] = intact(raw) and (out.float().cpu() - want).abs().max().item() <= 2e-3

# paged FP8 decode, Quest decode, metadata, append
Qp, Kp, Vp, _ = workloads.planted_block_cache(2, 8, 2, 2048, seed=5)
kc, ks = oracle.quantize_e4m3(Kp); vc, vs = oracle.quantize_e4m3(Vp)
perm = torch.randperm(2 * 128 + 3, generator=torch.Generator().manual_seed(1))
kpool, kspool, table = oracle.build_paged_cache(kc, ks, 16, perm)
vpool, vspool, _ = oracle.build_paged_cache(vc, vs, 16, perm)
plens = torch.tensor([2048, 777], dtype=torch.int32)
buf = paged.pack_fused(kpool.to(dev), vpool.to(dev), kspool.to(dev), vspool.to(dev))
kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table.to(dev), plens.to(dev), 2)
Kd, Vd = oracle.dequantize(kc, ks), oracle.dequantize(vc, vs)
raw, out = canary((2, 8, 128), torch.float16)
_C.fused_gqa_paged(Qp.to(dev), kv.k_pool, kv.v_pool, kv.k_scale, kv.v_scale, kv.page_table, kv.seq_lens, 128 ** -0.5, out=out)
want = oracle.dense_gqa_decode(Qp, Kd.permute(0, 2, 1, 3), Vd.permute(0, 2, 1, 3), 128 ** -0.5, plens)
ok["paged"] = intact(raw) and (out.float().cpu() - want).abs().max().item() <= 2e-3
meta = paged.build_block_meta(kv, 64)
qo, qi = paged.quest_sparse_decode(Qp.to(dev), kv, meta, 128 ** -0.5, 64, 4, return_indices=True)
want = oracle.attend_selected_blocks(Qp, Kd, Vd, qi.cpu().long(), 64, 128 ** -0.5, plens)
ok["quest"] = (qo.float().cpu() - want).abs().max().item() <= 2e-3
qkv = torch.randn(2, (8 + 4) * 128, generator=torch.Generator().manual_seed(2)).half().to(dev)
room = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table.to(dev), torch.tensor([100, 777], dtype=torch.int32, device=dev), 2)
ok["append"] = bool(torch.isfinite(paged.rope_quant_append(qkv, room, 8, 500000.0, meta=meta).float()).all())

# token-sparse and block-sparse decode (config-1 shape)
Qt, Kt, Vt = (t.half() for t in workloads.token_sparse_config1())
got = _C.token_sparse_decode(Qt.to(dev), Kt.to(dev), Vt.to(dev), 32, 4).float().cpu()
ok["token"] = (got - oracle.token_sparse_attention(Qt.float(), Kt.float(), Vt.float(), 32, 4)).abs().max().item() <= 2e-3
got = _C.sparse_attention_forward(Qt.to(dev), Kt.to(dev), Vt.to(dev), 64, 4).float().cpu()
ok["block"] = (got - oracle.block_sparse_mean_attention(Qt, Kt, Vt, 64, 4)[0]).abs().max().item() <= 2e-3

# eviction through the C-ABI with every output between canaries, both launch structures
Ke, Ve, sc = workloads.eviction(2, 2, 4096, 128, rounds=4, seed=3)
keep = lib.skv_kv_evict_keep_count(4096, 512, 64)
idx_want = oracle.eviction_keep_indices(sc, 512, 64)
codes_want, scales_want = oracle.quantize_int8(oracle.evict_gather(Ke, Ve, idx_want)[0])
Kd_, Vd_, sd_ = Ke.to(dev), Ve.to(dev), sc.to(dev)
for fused in (0, 1):
    lib.skv_kv_evict_set_fused(fused)
    r_i, idx = canary((2, 2, keep), torch.int32)
    r_k, ko = canary((2, 2, keep, 128), torch.int8)
    r_v, vo = canary((2, 2, keep, 128), torch.int8)
    r_s, kso = canary((2, 2, keep), torch.float32)
    r_t, vso = canary((2, 2, keep), torch.float32)
    rc = lib.skv_kv_evict_quant(Kd_.data_ptr(), Vd_.data_ptr(), sd_.data_ptr(), idx.data_ptr(), ko.data_ptr(), vo.data_ptr(),
                                kso.data_ptr(), vso.data_ptr(), 2, 2, 4096, 128, Kd_.stride(0), Kd_.stride(1), Kd_.stride(2),
                                512, 64, _lib.QUANT_INT8, _lib.ORDER_POSITION, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ok[f"evict_fused{fused}"] = (rc == 0 and all(intact(r) for r in (r_i, r_k, r_v, r_s, r_t))
                                 and torch.equal(idx.cpu().long(), idx_want) and torch.equal(ko.cpu(), codes_want)
                                 and torch.equal(kso.cpu(), scales_want))
lib.skv_kv_evict_set_fused(0)
torch.cuda.synchronize()
res["ok"] = ok
# after the self-test the file that holds it (skv_api) has a recorded line; every kernel file must be clean
res["violations"] = {n: word("skv_debug_bounds_" + n) for n in ("token_sparse", "block_sparse", "kv_evict", "paged_quest", "kv_append")}
print(json.dumps(res))
'''


def test_bounds_checked_library_runs_the_hot_path_without_a_violation(cuda_device):
    from llm_inference_optimization_b200 import build
    lib_path = build.build(bounds=True)
    env = dict(os.environ, SKV_B200_LIB=str(lib_path), PYTHONPATH=str(ROOT))
    proc = subprocess.run([sys.executable, "-c", DRIVER % {"root": str(ROOT)}], capture_output=True, text=True,
                          timeout=600, cwd=ROOT, env=env)
    assert proc.returncode == 0, proc.stderr[-3000:]
    res = json.loads([l for l in proc.stdout.splitlines() if l.startswith("{")][-1])
    assert res["lib"].endswith("libskv_b200_bounds.so")
    assert res["selftest"] == [2, 0, True]
    assert all(res["ok"].values()), res["ok"]
    assert all(v == 0 for v in res["violations"].values()), res["violations"]
