"""The weight-streaming GEMM of the decode step against a plain PyTorch fp32 matmul of the same 16-bit inputs."""
import pytest
import torch

from llm_inference_optimization_b200 import _workspace, glue

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,K,N", [(16, 4096, 6144), (16, 4096, 4096), (16, 14336, 4096), (16, 4096, 28672),   # tp1 layer
                                      (16, 4096, 768), (16, 512, 4096), (16, 1792, 4096), (16, 4096, 3584),       # tp8 slices
                                      (1, 128, 64), (3, 256, 192), (7, 1024, 64), (16, 128, 64 * 301), (5, 32, 320), (16, 8192 + 32, 448)])   # edges
def test_matches_fp32_matmul(cuda_device, dtype, rows, K, N):
    g = torch.Generator().manual_seed(rows * K + N)
    x = torch.randn(rows, K, generator=g).to(dtype)
    w = (torch.randn(K, N, generator=g) * 0.02).to(dtype)
    want = x.float() @ w.float()
    xd, wd = x.to(cuda_device), w.to(cuda_device)
    for _ in range(2):   # the second call finds the first call's partial sums and tickets in the workspace
        got = glue.skinny_gemm(xd, wd)
        torch.cuda.synchronize()
        assert _workspace.status(_workspace.get("skinny_gemm", 0, cuda_device)) == 0
        # the output is rounded to 16 bits once: half an ulp of the result plus fp32 summation-order noise
        tol = (2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -10) * want.abs().max().item() + 1e-5
        assert (got.float().cpu() - want).abs().max().item() <= tol


def test_writes_into_a_given_buffer_and_rejects_other_shapes(cuda_device):
    x = torch.randn(16, 256, device=cuda_device, dtype=torch.bfloat16)
    w = torch.randn(256, 128, device=cuda_device, dtype=torch.bfloat16)
    big = torch.zeros(3, 16, 128, device=cuda_device, dtype=torch.bfloat16)
    glue.skinny_gemm(x, w, out=big[1])
    assert (big[0] == 0).all() and (big[2] == 0).all()
    assert (big[1].float() - x.float() @ w.float()).abs().max().item() <= 2.0 ** -8 * 64
    assert not glue.skinny_gemm_supported(17, 256, 128) and not glue.skinny_gemm_supported(16, 200, 128)
    assert not glue.skinny_gemm_supported(16, 256, 96)
    with pytest.raises(RuntimeError):
        glue.skinny_gemm(torch.randn(17, 256, device=cuda_device, dtype=torch.bfloat16), w)
