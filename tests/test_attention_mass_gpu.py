"""Attention-mass output of the dense decode kernel and the eviction policy loop built on it."""
import pytest
import torch

from llm_inference_optimization_b200 import _C, eviction
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu


def make(B, Hq, Hkv, N, D, seed):
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(B, Hq, D, generator=g).half()
    K = torch.randn(B, N, Hkv, D, generator=g).half()
    V = torch.randn(B, N, Hkv, D, generator=g).half()
    return Q, K, V


@pytest.mark.parametrize("B,Hq,Hkv,N,D,lens", [(1, 32, 8, 4096, 128, None), (2, 8, 2, 3000, 128, [3000, 1234]),
                                               (1, 16, 1, 700, 64, [513]), (2, 4, 4, 257, 128, None)])
def test_mass_matches_oracle(cuda_device, B, Hq, Hkv, N, D, lens):
    Q, K, V = make(B, Hq, Hkv, N, D, seed=N)
    sl = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    scale = D ** -0.5
    mass = torch.full((B, Hkv, N), 0.25, dtype=torch.float32, device=cuda_device)   # accumulates on top of this
    out = _C.fused_gqa(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), scale,
                       seq_lens=None if sl is None else sl.to(cuda_device), mass=mass)
    torch.cuda.synchronize()
    want_out = oracle.dense_gqa_decode(Q, K, V, scale, sl)
    want = oracle.attention_mass(Q, K, scale, sl)
    assert (out.float().cpu() - want_out).abs().max().item() <= 2e-3       # the attention output is unchanged
    got = mass.cpu() - 0.25
    if sl is not None:                                                     # tokens past the end are not touched
        for b, n in enumerate(lens):
            assert torch.equal(mass[b, :, n:].cpu(), torch.full((Hkv, N - n), 0.25))
            got[b, :, n:] = 0
    assert (got - want).abs().max().item() <= 2e-5 + 1e-3 * want.abs().max().item()
    # every head's probabilities sum to one: the mass of a kv-head sums to its group size
    G = Hq // Hkv
    assert torch.allclose(got.sum(-1), torch.full((B, Hkv), float(G)), atol=2e-3)


def test_policy_loop_evicts_what_the_oracle_would(cuda_device):
    """Several decode steps accumulate mass; the kept set equals the oracle's top-k of the summed probabilities."""
    B, Hq, Hkv, N, D, steps, budget, recent = 1, 8, 2, 2048, 128, 4, 256, 16
    g = torch.Generator().manual_seed(21)
    K = torch.randn(B, N, Hkv, D, generator=g).half()
    V = torch.randn(B, N, Hkv, D, generator=g).half()
    pol = eviction.AttentionMassPolicy(B, Hkv, N, cuda_device)
    want = torch.zeros(B, Hkv, N)
    Kd, Vd = K.to(cuda_device), V.to(cuda_device)
    for _ in range(steps):
        Q = (torch.randn(B, Hq, D, generator=g) * 2).half()
        pol.decode(Q.to(cuda_device), Kd, Vd, D ** -0.5)
        want += oracle.attention_mass(Q, K, D ** -0.5)
    torch.cuda.synchronize()
    assert pol.steps == steps
    got_mass = pol.mass.cpu().clone()
    assert (got_mass - want).abs().max().item() <= 1e-4 + 1e-3 * want.max().item()
    res = pol.evict(Kd, Vd, budget, recent_tokens=recent, quant="int8", return_aux=True)
    torch.cuda.synchronize()
    # the kernel's own mass decides the set exactly; against the oracle's mass allow the few boundary swaps that
    # a 1e-3 relative difference in near-equal scores can cause
    keep_exact = oracle.eviction_keep_indices(got_mass, budget, recent)
    assert torch.equal(res.indices.cpu().long(), keep_exact.long())
    keep_oracle = oracle.eviction_keep_indices(want, budget, recent)
    for h in range(Hkv):
        a, b = set(res.indices[0, h].tolist()), set(keep_oracle[0, h].tolist())
        assert len(a ^ b) <= 6
    assert float(pol.mass.abs().max()) == 0.0 and pol.steps == 0


def test_evicted_cache_goes_back_into_pages(cuda_device):
    """Policy loop closed: mass-driven FP8 eviction, kept rows re-paged into an existing pool, paged decode over
    them equals dense attention over the dequantised kept rows."""
    from llm_inference_optimization_b200 import paged
    B, Hq, Hkv, N, D, budget, recent = 2, 8, 2, 1024, 128, 200, 24
    g = torch.Generator().manual_seed(5)
    K = torch.randn(B, N, Hkv, D, generator=g).half()
    V = torch.randn(B, N, Hkv, D, generator=g).half()
    pol = eviction.AttentionMassPolicy(B, Hkv, N, cuda_device)
    Kd, Vd = K.to(cuda_device), V.to(cuda_device)
    for _ in range(2):
        pol.decode((torch.randn(B, Hq, D, generator=g) * 2).half().to(cuda_device), Kd, Vd, D ** -0.5)
    res = pol.evict(Kd, Vd, budget, recent_tokens=recent, quant="fp8", return_aux=True)
    keep = res.K.shape[2]
    assert keep == budget + recent
    n = (keep + 15) // 16
    pool = torch.zeros(64, Hkv, paged.RECORD_ROWS, 128, dtype=torch.uint8, device=cuda_device)
    ids = torch.randperm(64, generator=g)[:B * n].view(B, n).to(cuda_device)
    kv = paged.repage_evicted(res, pool=pool, page_ids=ids)
    q = torch.randn(B, Hq, D, generator=g).half()
    got = kv.decode(q.to(cuda_device), D ** -0.5).float().cpu()
    Kq = oracle.dequantize(res.K.cpu(), res.k_scale.cpu())        # [B,Hkv,keep,D]
    Vq = oracle.dequantize(res.V.cpu(), res.v_scale.cpu())
    want = oracle.dense_gqa_decode(q, Kq.permute(0, 2, 1, 3), Vq.permute(0, 2, 1, 3), D ** -0.5)
    assert (got - want).abs().max().item() <= 2e-3
    # fresh storage instead of an existing pool gives the same answer
    got2 = paged.repage_evicted(res).decode(q.to(cuda_device), D ** -0.5).float().cpu()
    assert torch.equal(got, got2)
