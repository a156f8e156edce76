"""Decode-step glue kernels against plain torch fp32 arithmetic."""
import pytest
import torch

from llm_inference_optimization_b200 import _C, glue, paged

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hidden", [(16, 4096), (3, 8192), (1, 264)])
def test_residual_rmsnorm(cuda_device, dtype, rows, hidden):
    g = torch.Generator().manual_seed(rows * hidden)
    x = torch.randn(rows, hidden, generator=g).to(dtype).to(cuda_device)
    d = (torch.randn(rows, hidden, generator=g) * 0.3).to(dtype).to(cuda_device)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).to(cuda_device)
    want_resid = (x.float() + d.float()).to(dtype)                       # the sum is rounded to the storage type
    xf = want_resid.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float())
    resid = x.clone()
    out = glue.residual_rmsnorm(resid, d, w, 1e-5)
    torch.cuda.synchronize()
    assert torch.equal(resid, want_resid)
    ulp = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
    assert ((out.float() - want).abs() <= ulp * want.abs() + 1e-6).all()   # one rounding of the fp32 value
    # without a delta the residual stream is left alone
    resid2 = x.clone()
    out2 = glue.residual_rmsnorm(resid2, None, w, 1e-5)
    torch.cuda.synchronize()
    assert torch.equal(resid2, x)
    xf = x.float()
    want2 = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert ((out2.float() - want2).abs() <= ulp * want2.abs() + 1e-6).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_mul(cuda_device, dtype):
    g = torch.Generator().manual_seed(5)
    gu = (torch.randn(16, 2 * 14336, generator=g) * 2).to(dtype).to(cuda_device)
    out = glue.silu_mul(gu)
    torch.cuda.synchronize()
    gate, up = gu[:, :14336].float(), gu[:, 14336:].float()
    want = (torch.nn.functional.silu(gate).to(dtype).float() * up)
    ulp = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
    # silu is evaluated with the fast exponential: allow one more step of the storage type on the inner rounding
    assert ((out.float() - want).abs() <= 3 * ulp * want.abs() + 1e-6).all()


def test_glue_rejects_bad_shapes(cuda_device):
    x = torch.zeros(2, 100, dtype=torch.bfloat16, device=cuda_device)   # hidden not a multiple of 8
    with pytest.raises(RuntimeError):
        glue.residual_rmsnorm(x, None, torch.ones(100, dtype=torch.bfloat16, device=cuda_device), 1e-5)
    with pytest.raises(RuntimeError):
        glue.silu_mul(torch.zeros(2, 24, dtype=torch.bfloat16, device=cuda_device))


def test_paged_decode_bf16_output(cuda_device):
    """The bf16 output option stores the same fp32 result, rounded to bf16 instead of fp16."""
    B, Hq, Hkv, D, pages = 2, 32, 8, 128, 64
    g = torch.Generator().manual_seed(8)
    buf = torch.randint(0, 120, (pages, Hkv, paged.RECORD_ROWS, 128), generator=g, dtype=torch.uint8).to(cuda_device)
    table = torch.randperm(pages, generator=g)[:B * 32].view(B, 32).to(torch.int32).to(cuda_device)
    lens = torch.tensor([500, 311], dtype=torch.int32, device=cuda_device)
    kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table, lens, B)
    kv.k_scale.fill_(0.01)
    kv.v_scale.fill_(0.02)
    q = torch.randn(B, Hq, D, generator=g).half().to(cuda_device)
    o16 = _C.fused_gqa_paged(q, kv.k_pool, kv.v_pool, kv.k_scale, kv.v_scale, table, lens, D ** -0.5)
    obf = torch.empty(B, Hq, D, dtype=torch.bfloat16, device=cuda_device)
    _C.fused_gqa_paged(q, kv.k_pool, kv.v_pool, kv.k_scale, kv.v_scale, table, lens, D ** -0.5, out=obf)
    torch.cuda.synchronize()
    assert torch.isfinite(obf.float()).all()
    assert ((obf.float() - o16.float()).abs() <= 2.0 ** -8 * o16.float().abs() + 1e-3).all()
