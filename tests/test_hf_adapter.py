"""Hugging Face Llama adapter (the reference's patch_attention, benchmarks/llama_integration_benchmark.py:114-245)
on a small random-init model: prefill stays dense, decode steps go through the kernels."""
import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import LlamaConfig, LlamaForCausalLM  # noqa: E402

from llm_inference_optimization_b200 import hf_adapter  # noqa: E402


def small_model(dtype=torch.float32, device="cpu", head_dim=64):
    cfg = LlamaConfig(hidden_size=8 * head_dim, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, vocab_size=128, max_position_embeddings=4096)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).eval().to(device=device, dtype=dtype)


def test_patch_and_restore_bookkeeping():
    m = small_model()
    before = m.config._attn_implementation
    assert hf_adapter.patch_attention(m, mode="dense") == 2
    assert m.config._attn_implementation == hf_adapter.BACKEND
    assert hf_adapter.patch_attention(m, mode="token-sparse", sparse_layers=[1]) == 1   # re-patching keeps the original
    ids = torch.randint(0, 128, (1, 24))
    with torch.no_grad():
        out = m(ids, use_cache=True)                      # prefill: dense and causal through SDPA, also on CPU
        assert torch.isfinite(out.logits).all()
        with pytest.raises(RuntimeError):                 # a decode step needs the GPU: no silent fallback
            m(ids[:, :1], past_key_values=out.past_key_values, use_cache=True)
    assert hf_adapter.restore_attention(m) == 2
    assert m.config._attn_implementation == before
    assert hf_adapter.restore_attention(m) == 0
    with pytest.raises(ValueError):
        hf_adapter.patch_attention(m, mode="nope")
    with pytest.raises(ValueError):
        hf_adapter.patch_attention(m, sparse_layers=[7])


def _decode_logits(m, ids, nxt):
    with torch.no_grad():
        pre = m(ids, use_cache=True)
        return m(nxt, past_key_values=pre.past_key_values, use_cache=True).logits.float()


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim", [64, 128])
def test_decode_step_matches_sdpa(cuda_device, head_dim):
    """Dense mode, and sparse modes wide enough to keep every token, reproduce the stock model's next-token logits."""
    m = small_model(torch.float16, cuda_device, head_dim)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 128, (2, 320), generator=g).to(cuda_device)
    nxt = torch.randint(0, 128, (2, 1), generator=g).to(cuda_device)
    want = _decode_logits(m, ids, nxt)
    for kw in (dict(mode="dense"), dict(mode="token-sparse", top_k=321), dict(mode="dense", sparse_layers=[0])):
        hf_adapter.patch_attention(m, **kw)
        got = _decode_logits(m, ids, nxt)
        hf_adapter.restore_attention(m)
        assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3, kw
    # sparse modes that really drop tokens: finite logits of the right shape (the kernels' own parity is tested elsewhere)
    for kw in (dict(mode="token-sparse", top_k=32), dict(mode="block-sparse", block_size=64, top_k_blocks=2)):
        hf_adapter.patch_attention(m, **kw)
        got = _decode_logits(m, ids, nxt)
        hf_adapter.restore_attention(m)
        assert got.shape == want.shape and torch.isfinite(got).all()
