"""Token-sparse decode through the C-ABI vs the oracle and the reference-generated golden outputs."""
from pathlib import Path

import numpy as np
import pytest
import torch

import llm_inference_optimization_b200 as skv
from llm_inference_optimization_b200 import _C, workloads
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3
GOLDEN = Path(__file__).resolve().parent / "golden"


def boundary_gap(Q, K, top_k):
    """Smallest gap between the k-th and (k+1)-th score over all heads (fp32, fp16-rounded inputs)."""
    s = torch.matmul(Q.float(), K.float().transpose(-1, -2)) * Q.shape[-1] ** -0.5
    v = s.topk(min(top_k + 1, s.shape[-1]), -1).values
    return (v[..., top_k - 1] - v[..., top_k]).min().item() if top_k < s.shape[-1] else 1.0


@pytest.mark.parametrize("top_k,sink", [(256, 0), (256, 4), (32, 4)])
def test_config1_against_reference_golden(cuda_device, top_k, sink):
    """Config 1 (B=1,H=8,D=64,T=1024, seed 0): public API vs outputs of the reference's own function."""
    g = np.load(GOLDEN / "config1_token_sparse.npz")
    Q, K, V = workloads.token_sparse_config1()
    want = torch.from_numpy(g[f"out_h_k{top_k}_s{sink}"])  # reference evaluated on the fp16-rounded inputs
    got = skv.sparse_attention(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), top_k=top_k, sink_tokens=sink)
    assert got.dtype == torch.float32 and got.shape == (1, 8, 1, 64)
    assert (got.cpu() - want).abs().max().item() <= TOL


def test_topk_sets_bit_exact_config1(cuda_device):
    Q, K, V = workloads.token_sparse_config1()
    Qh, Kh, Vh = Q.half(), K.half(), V.half()
    assert boundary_gap(Qh, Kh, 256) > 1e-5
    _, idx = _C.token_sparse_decode(Qh.to(cuda_device), Kh.to(cuda_device), Vh.to(cuda_device), 256, 0,
                                    return_indices=True)
    want = oracle.token_topk_sets(Qh, Kh, 256)
    assert torch.equal(idx[:, :, 0].cpu().long(), want)


@pytest.mark.parametrize("B,H,T,D,k,sink", [(1, 32, 4096, 128, 32, 0), (2, 4, 1000, 128, 64, 4), (1, 2, 70000, 128, 512, 4),
                                            (1, 3, 50, 64, 64, 4), (2, 2, 333, 64, 1, 0), (1, 2, 5000, 128, 2048, 16)])
def test_shapes_against_oracle(cuda_device, B, H, T, D, k, sink):
    """Includes the reference's GPU test shape (1,32,4096,128,k=32), ragged T, top_k >= T and large k."""
    g = torch.Generator().manual_seed(B * 1000 + T)
    Q = torch.randn(B, H, 1, D, generator=g).half()
    K = torch.randn(B, H, T, D, generator=g).half()
    V = torch.randn(B, H, T, D, generator=g).half()
    out, idx = _C.token_sparse_decode(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), k, sink, return_indices=True)
    want = oracle.token_sparse_attention(Q.float(), K.float(), V.float(), k, sink)
    assert (out.float().cpu() - want).abs().max().item() <= TOL
    if boundary_gap(Q, K, k) > 1e-5:
        kk = min(k, T)
        assert torch.equal(idx[:, :, 0, :kk].cpu().long(), oracle.token_topk_sets(Q, K, k))
        assert (idx[:, :, 0, kk:] == -1).all()


def test_multi_query_rows(cuda_device):
    g = np.load(GOLDEN / "token_sparse_multiquery.npz")
    torch.manual_seed(11)
    Q, K, V = torch.randn(1, 8, 16, 64), torch.randn(1, 8, 512, 64), torch.randn(1, 8, 512, 64)
    got = skv.sparse_attention(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), 64, 4).cpu()
    want = oracle.token_sparse_attention(Q.half().float(), K.half().float(), V.half().float(), 64, 4)
    assert (got - want).abs().max().item() <= TOL
    assert (got - torch.from_numpy(g["out_h_k64_s4"])).abs().max().item() <= TOL  # reference on the fp16-rounded inputs


def test_tied_scores_resolve_to_lower_position(cuda_device):
    """Duplicate keys give exactly equal scores; the kept set must take the lower positions."""
    g = torch.Generator().manual_seed(1)
    Q = torch.randn(1, 1, 1, 64, generator=g).half()
    base = torch.randn(1, 1, 8, 64, generator=g).half()
    K = base.repeat(1, 1, 16, 1)  # 128 keys, every score value appears 16 times
    V = torch.randn(1, 1, 128, 64, generator=g).half()
    _, idx = _C.token_sparse_decode(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), 20, 0, return_indices=True)
    s = (K[0, 0].float() @ Q[0, 0, 0].float())
    order = torch.argsort(s, descending=True, stable=True)[:20].sort().values
    assert torch.equal(idx[0, 0, 0].cpu().long(), order)


def test_reference_binding_semantics(cuda_device):
    Q = torch.randn(1, 2, 1, 128).half().to(cuda_device)
    K = torch.randn(1, 2, 256, 128).half().to(cuda_device)
    out = skv.kv_evict_quant_forward(Q, K, K, 16, False)
    assert out.shape == (1, 2, 1, 128) and out.dtype == torch.float16
    with pytest.raises(RuntimeError, match="INT8"):
        skv.kv_evict_quant_forward(Q, K, K, 16, True)
    with pytest.raises(RuntimeError):
        skv.kv_evict_quant_forward(Q.float(), K, K, 16, False)
    with pytest.raises(RuntimeError):
        skv.sparse_attention(Q.cpu(), K.cpu(), K.cpu())


@pytest.mark.parametrize("B,H,T,D,k,sink", [(1, 32, 4096, 128, 32, 0), (2, 3, 33000, 128, 32, 4), (1, 4, 70001, 64, 256, 0),
                                            (1, 2, 40000, 128, 8, 2), (3, 2, 129, 64, 16, 0)])
def test_tensor_core_and_register_scoring_agree(cuda_device, B, H, T, D, k, sink):
    """Decode-shaped calls score the keys on the tensor cores (K streamed by TMA); switched off, the register-load
    kernel does it.  Same exact products, so the same top-k sets wherever the k-th gap is not a rounding tie, with and
    without the per-chunk candidate lists (T >= 32768), ragged T and strided (head-major view of a token-major) caches."""
    from llm_inference_optimization_b200 import _lib, _workspace
    lib = _lib.load()
    g = torch.Generator().manual_seed(T + D)
    Q = torch.randn(B, H, 1, D, generator=g).half()
    Kt = torch.randn(B, T, H, D, generator=g).half()          # token-major storage: K[b, h, t] is a strided view
    Vt = torch.randn(B, T, H, D, generator=g).half()
    K, V = Kt.permute(0, 2, 1, 3), Vt.permute(0, 2, 1, 3)
    res = {}
    try:
        for mode in (1, 0):
            assert lib.skv_token_sparse_set_mma_scores(mode) == 0
            res[mode] = _C.token_sparse_decode(Q.to(cuda_device), Kt.to(cuda_device).permute(0, 2, 1, 3),
                                               Vt.to(cuda_device).permute(0, 2, 1, 3), k, sink, return_indices=True)
            torch.cuda.synchronize()
            assert all(_workspace.status(w) == 0 for w in _workspace.all_of("token_sparse", cuda_device))
    finally:
        lib.skv_token_sparse_set_mma_scores(1)
    want = oracle.token_sparse_attention(Q.float(), K.float(), V.float(), k, sink)
    for mode in (1, 0):
        assert (res[mode][0].float().cpu() - want).abs().max().item() <= TOL, mode
    if boundary_gap(Q, K, k) > 1e-5:
        assert torch.equal(res[1][1], res[0][1])
        assert torch.equal(res[1][1][:, :, 0, :min(k, T)].cpu().long(), oracle.token_topk_sets(Q, K, k))


@pytest.mark.parametrize("H,T,k", [(4, 16384, 32), (2, 40000, 8), (3, 70001, 32), (1, 131072, 64), (1, 300000, 32)])
def test_staggered_and_equal_chunks_select_the_same_tokens(cuda_device, H, T, k):
    """The tensor-core scoring kernel cuts a row into chunks of unequal length by default; with equal chunks the scores
    are the same numbers, so outputs and indices are identical bit for bit."""
    from llm_inference_optimization_b200 import _lib, _workspace
    lib = _lib.load()
    g = torch.Generator().manual_seed(T)
    Q = torch.randn(1, H, 1, 128, generator=g).half().to(cuda_device)
    K = torch.randn(1, H, T, 128, generator=g).half().to(cuda_device)
    V = torch.randn(1, H, T, 128, generator=g).half().to(cuda_device)
    res = {}
    try:
        for mode in (1, 0):
            assert lib.skv_token_sparse_set_stagger(mode) == 0
            res[mode] = _C.token_sparse_decode(Q, K, V, k, 0, return_indices=True)
            torch.cuda.synchronize()
            assert all(_workspace.status(w) == 0 for w in _workspace.all_of("token_sparse", cuda_device))
    finally:
        lib.skv_token_sparse_set_stagger(1)
    assert torch.equal(res[1][0], res[0][0])
    assert torch.equal(res[1][1], res[0][1])
    if boundary_gap(Q.cpu(), K.cpu(), k) > 1e-5:
        assert torch.equal(res[1][1][:, :, 0, :k].cpu().long(), oracle.token_topk_sets(Q.cpu(), K.cpu(), k))


@pytest.mark.parametrize("T,k", [(2000, 32), (4096, 100), (40000, 32)])
def test_equal_and_sorted_scores(cuda_device, T, k):
    """Rows the selection's shortcut cannot thin out: all scores equal (every element reaches any threshold; the kept
    set is the first k positions) and scores rising with the position (the k best sit in one thread group)."""
    g = torch.Generator().manual_seed(T)
    Q = torch.zeros(1, 2, 1, 64).half()
    Q[..., 0] = 1.0
    K = torch.zeros(1, 2, T, 64).half()
    K[0, 0, :, 0] = 0.5                                               # head 0: all equal
    K[0, 1, :, 0] = (torch.arange(T).float() / T).half()              # head 1: non-decreasing, runs of equal values
    K[..., 1:] = torch.randn(1, 2, T, 63, generator=g).half()         # orthogonal to q
    V = torch.randn(1, 2, T, 64, generator=g).half()
    out, idx = _C.token_sparse_decode(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), k, 0, return_indices=True)
    s = (K.float() @ Q.float().transpose(-1, -2))[..., 0]             # [1, 2, T]
    for h in range(2):
        want = torch.argsort(s[0, h], descending=True, stable=True)[:k].sort().values
        assert torch.equal(idx[0, h, 0].cpu().long(), want), h
        # (the oracle's torch.topk breaks ties its own way: attend over the expected set directly)
        w = torch.softmax(s[0, h, want] * 64 ** -0.5, dim=0)
        assert (out[0, h, 0].float().cpu() - w @ V[0, h, want].float()).abs().max().item() <= TOL
