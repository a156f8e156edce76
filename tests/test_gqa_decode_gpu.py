"""Dense GQA decode through the C-ABI vs the CPU oracle (max-abs <= 2e-3, fp32 accumulation)."""
import math

import pytest
import torch

from llm_inference_optimization_b200 import _C, _workspace, workloads
from oracle import skv_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3  # max-abs bound on attention outputs


def run(Q, K, V, scale, dev, seq_lens=None):
    lens = None if seq_lens is None else seq_lens.to(dev)
    out = _C.fused_gqa(Q.to(dev), K.to(dev), V.to(dev), scale, seq_lens=lens)
    torch.cuda.synchronize()
    assert _workspace.status(_workspace.get("gqa", 0, dev)) == 0
    return out.float().cpu()


@pytest.mark.parametrize("N", [4096, 16384, 65536])
def test_config2_llama_layer_shape(cuda_device, N):
    Q, K, V, scale = workloads.dense_gqa(N)
    got = run(Q, K, V, scale, cuda_device)
    want = oracle.dense_gqa_decode(Q, K, V, scale)
    assert (got - want).abs().max().item() <= TOL


@pytest.mark.parametrize("N", [1, 7, 63, 64, 65, 127, 1000, 4097, 64000])
def test_ragged_lengths(cuda_device, N):
    Q, K, V, scale = workloads.dense_gqa(N, seed=100 + N % 97)
    got = run(Q, K, V, scale, cuda_device)
    want = oracle.dense_gqa_decode(Q, K, V, scale)
    assert (got - want).abs().max().item() <= TOL


@pytest.mark.parametrize("B,Hq,Hkv,D", [(2, 8, 8, 128), (3, 16, 2, 128), (1, 8, 1, 64), (2, 32, 2, 64), (4, 12, 4, 128)])
def test_group_sizes_and_head_dims(cuda_device, B, Hq, Hkv, D):
    Q, K, V, scale = workloads.dense_gqa(777, B=B, Hq=Hq, Hkv=Hkv, D=D, seed=9)
    got = run(Q, K, V, scale, cuda_device)
    want = oracle.dense_gqa_decode(Q, K, V, scale)
    assert (got - want).abs().max().item() <= TOL


def test_unit_variance_inputs(cuda_device):
    g = torch.Generator().manual_seed(3)
    Q = torch.randn(1, 32, 128, generator=g).half()
    K = torch.randn(1, 8192, 8, 128, generator=g).half()
    V = torch.randn(1, 8192, 8, 128, generator=g).half()
    got = run(Q, K, V, 1 / math.sqrt(128), cuda_device)
    want = oracle.dense_gqa_decode(Q, K, V, 1 / math.sqrt(128))
    assert (got - want).abs().max().item() <= TOL


def test_seq_lens_and_strided_cache(cuda_device):
    """Per-sequence lengths, and a [B,Hkv,N,D] cache passed as a permuted view (no copy)."""
    B, N = 3, 3000
    Q, K, V, scale = workloads.dense_gqa(N, B=B, seed=21)
    lens = torch.tensor([3000, 1, 1537], dtype=torch.int32)
    Kc = K.permute(0, 2, 1, 3).contiguous().to(cuda_device)  # [B,Hkv,N,D] as an HF cache stores it
    Vc = V.permute(0, 2, 1, 3).contiguous().to(cuda_device)
    out = _C.fused_gqa(Q.to(cuda_device), Kc.permute(0, 2, 1, 3), Vc.permute(0, 2, 1, 3), scale,
                       seq_lens=lens.to(cuda_device))
    want = oracle.dense_gqa_decode(Q, K, V, scale, lens)
    assert (out.float().cpu() - want).abs().max().item() <= TOL


def test_repeated_calls_reuse_workspace(cuda_device):
    Q, K, V, scale = workloads.dense_gqa(20000, seed=5)
    want = oracle.dense_gqa_decode(Q, K, V, scale)
    Qd, Kd, Vd = Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device)
    for _ in range(5):
        got = _C.fused_gqa(Qd, Kd, Vd, scale).float().cpu()
        assert (got - want).abs().max().item() <= TOL


def test_split_invariance_full_size(cuda_device):
    """At 128K the result must not depend on how the KV length is split (1 vs 2 CTAs per SM)."""
    from llm_inference_optimization_b200 import _lib
    Q, K, V, scale = workloads.dense_gqa(131072, seed=1)
    Qd, Kd, Vd = Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device)
    lib = _lib.load()
    outs = []
    try:
        for stages, per_sm in ((6, 1), (3, 2), (2, 2)):
            _lib.check(lib.skv_gqa_set_tuning(stages, per_sm), "tuning")
            outs.append(_C.fused_gqa(Qd, Kd, Vd, scale).float().cpu())
    finally:
        lib.skv_gqa_set_tuning(4, 1)
    want = oracle.dense_gqa_decode(Q, K, V, scale)
    for o in outs:
        assert (o - want).abs().max().item() <= TOL
    assert (outs[0] - outs[1]).abs().max().item() <= 1e-3


def test_rejects_bad_arguments(cuda_device):
    Q, K, V, scale = workloads.dense_gqa(128)
    Qd, Kd, Vd = Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device)
    with pytest.raises(RuntimeError):
        _C.fused_gqa(Qd.float(), Kd, Vd, scale)
    with pytest.raises(RuntimeError):
        _C.fused_gqa(Qd[:, :30].contiguous(), Kd, Vd, scale)  # 30 % 8 != 0
    with pytest.raises(RuntimeError):
        _C.fused_gqa(Qd, Kd, Vd[:, :64], scale)
    with pytest.raises(RuntimeError):
        _C.fused_gqa(Q, K, V, scale)  # CPU tensors


@pytest.mark.parametrize("early", [0, 1])
def test_back_to_back_launches_both_launch_orders(cuda_device, early):
    """Eight launches over different static caches without a sync in between, in the default (fully ordered) mode
    and with early K/V streaming switched on: every launch still returns its own cache's attention."""
    from llm_inference_optimization_b200 import _lib
    cases = [workloads.dense_gqa(6000 + 500 * i, seed=40 + i) for i in range(8)]
    dev = [(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), s) for Q, K, V, s in cases]
    outs = [torch.empty_like(d[0]) for d in dev]
    lib = _lib.load()
    assert lib.skv_gqa_set_early_kv(early) == 0
    try:
        for _ in range(3):
            for (Q, K, V, s), o in zip(dev, outs):
                _C.fused_gqa(Q, K, V, s, out=o)
        torch.cuda.synchronize()
    finally:
        lib.skv_gqa_set_early_kv(0)
    assert _workspace.status(_workspace.get("gqa", 0, cuda_device)) == 0
    for (Q, K, V, s), o in zip(cases, outs):
        assert (o.float().cpu() - oracle.dense_gqa_decode(Q, K, V, s)).abs().max().item() <= 2e-3


@pytest.mark.parametrize("B,Hq,Hkv,N,lens", [(4, 8, 2, 6000, [6000, 1, 0, 3333]), (2, 32, 8, 9000, [9000, 4097]),
                                             (6, 4, 1, 2048, [2048, 2048, 64, 65, 1000, 7])])
def test_ragged_batch_work_list_schedule(cuda_device, lib, B, Hq, Hkv, N, lens):
    """With seq_lens and few (sequence, kv-head) pairs the fp16 kernel schedules from a work list derived from the
    real lengths (one wave of nearly equal CTAs); switched off it uses the host's plan for the longest sequence.
    Both must give the oracle's result, also with an empty and a one-token sequence, and the attention-mass output."""
    Q, K, V, scale = workloads.dense_gqa(N, B=B, Hq=Hq, Hkv=Hkv, seed=N)
    sl = torch.tensor(lens, dtype=torch.int32)
    want = oracle.dense_gqa_decode(Q, K, V, scale, sl)
    try:
        for mode in (1, 0):
            assert lib.skv_gqa_set_ragged_worklist(mode) == 0
            got = run(Q, K, V, scale, cuda_device, sl)
            assert (got - want).abs().max().item() <= TOL, mode
            mass = torch.zeros(B, Hkv, N, dtype=torch.float32, device=cuda_device)
            _C.fused_gqa(Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device), scale, seq_lens=sl.to(cuda_device), mass=mass)
            assert (mass.cpu() - oracle.attention_mass(Q, K, scale, sl)).abs().max().item() <= 1e-3, mode
    finally:
        lib.skv_gqa_set_ragged_worklist(1)


@pytest.mark.parametrize("B,Hq,Hkv,D,N,lens", [
    (1, 32, 8, 128, 4096, None), (1, 32, 8, 128, 16384, None), (1, 32, 8, 128, 24576, None),   # config-2 short contexts
    (2, 32, 8, 128, 8192, [8192, 130]), (3, 16, 2, 128, 5000, [5000, 0, 1]),                  # ragged, empty, one token
    (1, 8, 1, 64, 3000, None), (16, 32, 8, 128, 4096, None), (1, 16, 1, 128, 2048, None)])    # D = 64, many pairs, G = 16
def test_short_context_cluster_combine(cuda_device, lib, B, Hq, Hkv, D, N, lens):
    """Short contexts launch the splits of a (batch, kv-head) as one thread-block cluster and sum them through
    distributed shared memory; switched off, the same call goes through global-memory partials and the ticket.
    Both give the oracle's result, and they agree with each other to fp16 rounding."""
    Q, K, V, scale = workloads.dense_gqa(N, B=B, Hq=Hq, Hkv=Hkv, D=D, seed=N + B)
    sl = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    want = oracle.dense_gqa_decode(Q, K, V, scale, sl)
    got = {}
    try:
        for mode in (1, 0):
            assert lib.skv_gqa_set_cluster_combine(mode) == 0
            for _ in range(2):
                got[mode] = run(Q, K, V, scale, cuda_device, sl)
            assert (got[mode] - want).abs().max().item() <= TOL, mode
    finally:
        lib.skv_gqa_set_cluster_combine(1)
    assert (got[1] - got[0]).abs().max().item() <= 2.0 ** -10 * max(1.0, want.abs().max().item())
