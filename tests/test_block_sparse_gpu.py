"""Block-sparse decode (the reference's block-mean rule) through the C-ABI vs the oracle."""
import pytest
import torch

from llm_inference_optimization_b200 import _C, workloads
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def gap(Q, K, bs, k):
    sc = oracle.block_mean_scores(Q, K, bs)
    if k >= sc.shape[-1]:
        return 1.0
    v = sc.topk(k + 1, -1).values
    return (v[..., k - 1] - v[..., k]).min().item()


def check(cuda_device, Q, K, V, bs, k):
    out, idx = _C.sparse_attention_forward(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), bs, k,
                                           return_indices=True)
    want, blocks = oracle.block_sparse_mean_attention(Q, K, V, bs, k)
    assert out.shape == Q.shape and out.dtype == torch.float16
    assert (out.float().cpu() - want).abs().max().item() <= TOL
    if gap(Q, K, bs, k) > 1e-6:
        kk = blocks.shape[-1]
        assert torch.equal(idx[..., :kk].cpu().long(), blocks)   # block sets bit-exact
        assert (idx[..., kk:] == -1).all()


def test_config1_block_path(cuda_device):
    """B=1,H=8,D=64,T=1024, block 64, top 4 blocks, seed 0 (fp16-rounded inputs)."""
    Q, K, V = (t.half() for t in workloads.token_sparse_config1())
    check(cuda_device, Q, K, V, 64, 4)


@pytest.mark.parametrize("B,H,T,D,bs,k", [(1, 4, 300, 64, 64, 4),      # ragged tail (the reference's T=300 case)
                                          (1, 2, 256, 128, 64, 99),     # more blocks asked than exist
                                          (2, 8, 4096, 128, 64, 8),
                                          (1, 32, 65536, 128, 64, 8),   # 64K context, 1024 blocks
                                          (1, 2, 1000, 32, 16, 128),
                                          (1, 1, 40, 128, 64, 1)])      # a single partial block
def test_shapes(cuda_device, B, H, T, D, bs, k):
    g = torch.Generator().manual_seed(T + D)
    Q = torch.randn(B, H, 1, D, generator=g).half()
    K = torch.randn(B, H, T, D, generator=g).half()
    V = torch.randn(B, H, T, D, generator=g).half()
    check(cuda_device, Q, K, V, bs, k)


@pytest.mark.parametrize("B,H,T,D,bs,k", [(1, 32, 65536, 128, 64, 8), (2, 3, 5000, 128, 16, 8), (1, 2, 9000, 64, 48, 4),
                                          (1, 4, 300, 64, 64, 4), (1, 2, 40000, 128, 256, 3), (1, 1, 40, 128, 64, 1)])
def test_tensor_core_and_register_scoring_agree(cuda_device, B, H, T, D, bs, k):
    """The block scores come from the tensor-core kernel (sum of the tokens' scores over their count) or, switched off,
    from the register-load kernel: both against the oracle, with ragged tails, block sizes that do not divide the
    128-token tile, and a token-major cache viewed head-major (strided rows)."""
    from llm_inference_optimization_b200 import _lib, _workspace
    lib = _lib.load()
    g = torch.Generator().manual_seed(T + bs)
    Q = torch.randn(B, H, 1, D, generator=g).half()
    Kt = torch.randn(B, T, H, D, generator=g).half()
    Vt = torch.randn(B, T, H, D, generator=g).half()
    K, V = Kt.permute(0, 2, 1, 3), Vt.permute(0, 2, 1, 3)
    want, blocks = oracle.block_sparse_mean_attention(Q, K, V, bs, k)
    res = {}
    try:
        for mode in (1, 0):
            assert lib.skv_block_sparse_set_mma_scores(mode) == 0
            res[mode] = _C.sparse_attention_forward(Q.to(cuda_device), Kt.to(cuda_device).permute(0, 2, 1, 3),
                                                    Vt.to(cuda_device).permute(0, 2, 1, 3), bs, k, return_indices=True)
            torch.cuda.synchronize()
            assert all(_workspace.status(w) == 0 for w in _workspace.all_of("block_sparse", cuda_device))
            assert (res[mode][0].float().cpu() - want).abs().max().item() <= TOL, mode
    finally:
        lib.skv_block_sparse_set_mma_scores(1)
    if gap(Q, K, bs, k) > 1e-6:
        kk = blocks.shape[-1]
        assert torch.equal(res[1][1], res[0][1])
        assert torch.equal(res[1][1][..., :kk].cpu().long(), blocks)


def test_deterministic(cuda_device):
    g = torch.Generator().manual_seed(5)
    Q, K, V = (torch.randn(s, generator=g).half().to(cuda_device) for s in ((1, 4, 1, 128), (1, 4, 2048, 128), (1, 4, 2048, 128)))
    a = _C.sparse_attention_forward(Q, K, V, 64, 8)
    b = _C.sparse_attention_forward(Q, K, V, 64, 8)
    assert torch.equal(a, b) and torch.isfinite(a.float()).all()


def test_argument_errors(cuda_device):
    Q = torch.zeros(1, 2, 1, 64, dtype=torch.float16, device=cuda_device)
    K = torch.zeros(1, 2, 128, 64, dtype=torch.float16, device=cuda_device)
    with pytest.raises(RuntimeError, match="decode-step"):
        _C.sparse_attention_forward(Q.expand(1, 2, 2, 64), K, K, 64, 2)
    with pytest.raises(RuntimeError, match="top_k_blocks"):
        _C.sparse_attention_forward(Q, K, K, 64, 0)
    with pytest.raises(RuntimeError, match="block_size"):
        _C.sparse_attention_forward(Q, K, K, 0, 2)
    with pytest.raises(RuntimeError, match="fp16"):
        _C.sparse_attention_forward(Q.float(), K, K, 64, 2)
