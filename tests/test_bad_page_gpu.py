"""A page-table entry outside the pool is never turned into an address: the kernels read page 0 (or store nothing)
and set SKV_DEV_BAD_PAGE in the status word.  No kernel traps, and the output stays finite."""
import pytest
import torch

from llm_inference_optimization_b200 import _workspace, paged, workloads
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
SKV_DEV_BAD_PAGE = 2


def small_cache(dev, fused, lens=None):
    Q, K, V, _ = workloads.planted_block_cache(2, 8, 2, 1024, seed=41)
    kc, ks = oracle.quantize_e4m3(K)
    vc, vs = oracle.quantize_e4m3(V)
    perm = torch.randperm(2 * 64 + 5, generator=torch.Generator().manual_seed(3))
    kp, ksp, table = oracle.build_paged_cache(kc, ks, 16, perm)
    vp, vsp, _ = oracle.build_paged_cache(vc, vs, 16, perm)
    if fused:
        buf = paged.pack_fused(kp.to(dev), vp.to(dev), ksp.to(dev), vsp.to(dev))
        kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table.to(dev), lens, 2)
    else:
        kv = paged.PagedKV(kp.to(dev), vp.to(dev), ksp.to(dev), vsp.to(dev), table.to(dev), lens, 2)
    return Q, kv, kp.shape[0]


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("bad", [-1, 1 << 20, 2 ** 31 - 1])
def test_dense_paged_decode_reports_a_bad_page(cuda_device, fused, bad):
    Q, kv, num_pages = small_cache(cuda_device, fused)
    good = kv.decode(Q.to(cuda_device), 128 ** -0.5)
    ws = _workspace.get("gqa", 0, cuda_device)
    assert _workspace.status(ws) == 0
    kv.page_table[1, 7] = bad
    try:
        out = kv.decode(Q.to(cuda_device), 128 ** -0.5)
        assert _workspace.status(ws) & SKV_DEV_BAD_PAGE
        assert torch.isfinite(out.float()).all()
        assert torch.equal(out[0], good[0])          # the other sequence is untouched
    finally:
        ws.zero_()                                    # the status word is sticky until the owner clears it
        torch.cuda.synchronize()
    assert _workspace.status(ws) == 0


def test_quest_decode_and_meta_report_a_bad_page(cuda_device):
    Q, kv, num_pages = small_cache(cuda_device, True)
    kv.page_table[0, 3] = num_pages + 11
    st = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    meta = paged.build_block_meta(kv, 64, status=st)
    assert int(st.item()) & SKV_DEV_BAD_PAGE and torch.isfinite(meta.float()).all()
    kv.page_table[0, :] = num_pages + 11              # whatever blocks are chosen, their pages are bad
    ws = _workspace.get("quest", 0, cuda_device)
    try:
        out = paged.quest_sparse_decode(Q.to(cuda_device), kv, meta, 128 ** -0.5, 64, 4)
        assert _workspace.status(ws) & SKV_DEV_BAD_PAGE
        assert torch.isfinite(out.float()).all()
    finally:
        ws.zero_()
        torch.cuda.synchronize()


def test_append_stores_nothing_through_a_bad_page(cuda_device):
    B, Hq, Hkv, D, pages = 2, 8, 2, 128, 40
    g = torch.Generator().manual_seed(7)
    table = torch.randperm(pages, generator=g)[:B * 16].view(B, 16).to(torch.int32).to(cuda_device)
    table[1, 0] = pages                               # first page of sequence 1 lies one past the pool
    buf = torch.zeros(pages, Hkv, paged.RECORD_ROWS, 128, dtype=torch.uint8, device=cuda_device)
    guard = torch.zeros_like(buf)                     # allocated right behind: a stray store would likely land here
    lens = torch.zeros(B, dtype=torch.int32, device=cuda_device)
    kv = paged.PagedKV.from_fused(buf, torch.float8_e4m3fn, table, lens, B)
    st = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).half().to(cuda_device)
    q = paged.rope_quant_append(qkv, kv, Hq, 500000.0, status=st)
    assert int(st.item()) & SKV_DEV_BAD_PAGE and torch.isfinite(q.float()).all()
    assert (guard == 0).all()
    touched = buf.flatten(1).any(dim=1).nonzero().flatten().tolist()
    assert touched == [int(table[0, 0])]              # only sequence 0 stored its token
