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
    # the order torch.topk returns: all 4160 kept rows by descending score (the recent window carries +inf in the
    # selection but is ordered here by its real scores), equal scores by ascending position
    order_idx = rs.indices.cpu().long()
    s_sorted = torch.gather(scores, 2, order_idx)
    assert (s_sorted[..., :-1] >= s_sorted[..., 1:]).all()
    ties = s_sorted[..., :-1] == s_sorted[..., 1:]
    assert (order_idx[..., :-1][ties] < order_idx[..., 1:][ties]).all()
    want_order = torch.gather(idx, 2, torch.sort(torch.gather(scores, 2, idx), dim=-1, descending=True, stable=True).indices)
    assert torch.equal(order_idx, want_order)


@pytest.mark.parametrize("quant", ["int8", "fp8", "none"])
@pytest.mark.parametrize("B,H,T,D,budget,recent", [(4, 8, 32768, 128, 4096, 64), (2, 3, 5000, 64, 300, 7),
                                                   (1, 2, 96, 128, 10, 90), (1, 1, 40, 128, 64, 0)])
def test_single_launch_and_two_launch_paths_agree(cuda_device, lib, quant, B, H, T, D, budget, recent):
    """The cluster kernel that selects and gathers in one launch against the select + gather launches: bit-identical."""
    K, V, scores = workloads.eviction(B, H, T, D, rounds=4, seed=T + 1)
    Kd, Vd, sd = K.to(cuda_device), V.to(cuda_device), scores.to(cuda_device)
    kw = dict(recent_tokens=recent, return_aux=True)
    kw.update(dict(use_int8=False, order="position") if quant == "none" else dict(quant=quant))
    try:
        assert lib.skv_kv_evict_set_fused(1) == 0
        one = skv.fused_kv_evict(Kd, Vd, sd, budget, **kw)
        assert lib.skv_kv_evict_set_fused(0) == 0
        two = skv.fused_kv_evict(Kd, Vd, sd, budget, **kw)
    finally:
        lib.skv_kv_evict_set_fused(0)
    assert torch.equal(one.indices, two.indices)
    assert torch.equal(one.indices.cpu().long(), oracle.eviction_keep_indices(scores, budget, recent))
    assert torch.equal(one.K.view(torch.uint8), two.K.view(torch.uint8)) and torch.equal(one.V.view(torch.uint8), two.V.view(torch.uint8))
    if quant != "none":
        assert torch.equal(one.k_scale, two.k_scale) and torch.equal(one.v_scale, two.v_scale)
