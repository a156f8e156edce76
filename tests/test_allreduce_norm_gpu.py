"""Fused all-reduce + residual + RMSNorm kernel.  On one GPU the peers are emulated by local buffers whose flags
the test sets by hand (the kernel never waits on another launch); two real ranks run in the decode-step test."""
import os
import socket

import pytest
import torch

from llm_inference_optimization_b200 import decode_step as ds, glue
from llm_inference_optimization_b200.sharding import shard_heads

pytestmark = pytest.mark.gpu


def _peers(world, rows, hidden, dtype, dev, g):
    bufs = []
    for _ in range(2):
        bufs.append([((torch.randn(rows, hidden, generator=g) * 0.5).to(dtype).to(dev),
                      torch.zeros(glue.AllReduceNorm.FLAG_WORDS, dtype=torch.int32, device=dev)) for _ in range(world)])
    for r in range(world):          # one flag array per rank, shared by both buffers
        bufs[1][r] = (bufs[1][r][0], bufs[0][r][1])
    return bufs


def _want(parts, resid, w, eps, dtype):
    acc = parts[0].float()
    for p in parts[1:]:
        acc = acc + p.float()
    x = (resid.float() + acc.to(dtype).float()).to(dtype)
    xf = x.float()
    return x, xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_emulated_peers_sum_and_normalise(cuda_device, dtype, world):
    rows, hidden = 16, 4096
    g = torch.Generator().manual_seed(world)
    peers = _peers(world, rows, hidden, dtype, cuda_device, g)
    arn = glue.AllReduceNorm(rows, hidden, dtype, cuda_device, peers=peers, rank=0, max_spins=2000)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).to(cuda_device)
    resid = torch.randn(rows, hidden, generator=g).to(dtype).to(cuda_device)
    ulp = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
    for call in range(3):                                   # epochs 1, 2, 3 on alternating buffers
        i = call % 2
        for r in range(1, world):
            peers[0][0][1][r] = call + 1                    # "peer r says: my partial of this epoch is complete"
        before = resid.clone()
        out = arn.reduce_norm(i, resid, w, 1e-5)
        torch.cuda.synchronize()
        want_resid, want = _want([p[0] for p in peers[i]], before, w, 1e-5, dtype)
        assert arn.status() == 0
        assert torch.equal(resid, want_resid)
        assert ((out.float() - want).abs() <= ulp * want.abs() + 1e-6).all()
        assert int(peers[0][0][1][0]) == call + 1           # the kernel signalled its own epoch
        assert int(arn.sync[0]) == call + 1 and int(arn.sync[1]) == 0


def test_missing_peer_times_out_and_recovers(cuda_device):
    """A peer that never signals: the bounded wait runs out, the status word says so, nothing is stored, and the
    context stays usable for the next call."""
    rows, hidden, dtype = 4, 1024, torch.bfloat16
    g = torch.Generator().manual_seed(3)
    peers = _peers(2, rows, hidden, dtype, cuda_device, g)
    arn = glue.AllReduceNorm(rows, hidden, dtype, cuda_device, peers=peers, rank=0, max_spins=500)
    w = torch.ones(hidden, dtype=dtype, device=cuda_device)
    resid = torch.randn(rows, hidden, generator=g).to(dtype).to(cuda_device)
    before = resid.clone()
    arn.reduce_norm(0, resid, w, 1e-5)                       # peer 1's flag is still 0
    torch.cuda.synchronize()
    assert arn.status() == 1
    assert torch.equal(resid, before)
    assert int(arn.sync[0]) == 1                             # the epoch still advances: later calls stay in step
    arn.sync[2] = 0
    peers[0][0][1][1] = 2
    out = arn.reduce_norm(1, resid, w, 1e-5)
    torch.cuda.synchronize()
    want_resid, want = _want([p[0] for p in peers[1]], before, w, 1e-5, dtype)
    assert arn.status() == 0 and torch.equal(resid, want_resid)
    assert ((out.float() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-6).all()


def test_rejects_bad_arguments(cuda_device):
    g = torch.Generator().manual_seed(1)
    peers = _peers(3, 2, 64, torch.bfloat16, cuda_device, g)
    arn = glue.AllReduceNorm(2, 64, torch.bfloat16, cuda_device, peers=peers, rank=0)
    with pytest.raises(RuntimeError):                        # world of 3 is not supported
        arn.reduce_norm(0, torch.zeros(2, 64, dtype=torch.bfloat16, device=cuda_device),
                        torch.ones(64, dtype=torch.bfloat16, device=cuda_device), 1e-5)


CFG = ds.ModelConfig(layers=2, hidden=512, Hq=8, Hkv=2, D=128, mlp=1024, vocab=256)
LENS = torch.tensor([700, 33, 1500], dtype=torch.int32)
TOK = torch.tensor([5, 77, 200])


def _tp_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        outs = []
        for fused in (False, "pull", "push"):
            m = ds.DecodeModel(CFG, shard_heads(CFG.Hq, CFG.Hkv, world, rank), dev, dtype=torch.bfloat16)
            m.init_cache(LENS, fill="normal")
            if fused:
                m.enable_fused_allreduce(len(TOK), protocol=fused)
            for _ in range(3):
                out = m.step(TOK.cuda())
            torch.cuda.synchronize()
            outs.append(out.float().cpu().numpy())
            if fused and m.arn.status() != 0:
                raise RuntimeError("a peer wait ran out")
        if rank == 0:
            ret.put(outs)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_decode_step_without_nccl_allreduce(cuda_device):
    """bf16 decode steps on two ranks: the fused peer-memory all-reduce gives the logits of the NCCL path."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    nccl, pull, push = (torch.from_numpy(a) for a in ret.get(timeout=300))
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for fused in (pull, push):
        cos = torch.nn.functional.cosine_similarity(nccl, fused, dim=-1)
        assert cos.min().item() > 0.999
        assert (nccl - fused).abs().max().item() <= 3e-2 * nccl.abs().max().item()
    assert torch.equal(pull, push)       # both protocols sum the ranks' rows in rank order


def _ll_words(part, epoch):
    """[rows, hidden] 16-bit values -> the 8-byte words a pushing rank writes: 4 bytes of data, then the epoch."""
    data = part.contiguous().view(torch.int32).reshape(-1)              # two 16-bit values per word
    return torch.stack((data, torch.full_like(data, epoch)), dim=1).reshape(-1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_push_protocol_with_emulated_peers(cuda_device, dtype, world):
    """The push variant: the peers' rows arrive in this rank's receive region as (data, epoch) words -- written by the
    test here -- and this rank's own row goes out into every peer's region the same way."""
    rows, hidden = 16, 4096
    g = torch.Generator().manual_seed(10 + world)
    region = world * rows * hidden * 4
    recv = [[torch.zeros(region, dtype=torch.uint8, device=cuda_device) for _ in range(world)] for _ in range(2)]
    arn = glue.AllReduceNorm(rows, hidden, dtype, cuda_device, push_peers=recv, rank=0, max_spins=2000, protocol="push")
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).to(cuda_device)
    resid = torch.randn(rows, hidden, generator=g).to(dtype).to(cuda_device)
    ulp = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
    per_src = rows * hidden // 2 * 2                                     # int32 words per source rank
    for call in range(3):
        i, epoch = call % 2, call + 1
        parts = [(torch.randn(rows, hidden, generator=g) * 0.5).to(dtype).to(cuda_device) for _ in range(world)]
        arn.partial(i).copy_(parts[0])
        mine = recv[i][0].view(torch.int32)
        for r in range(1, world):                                        # "peer r has pushed its row of this epoch"
            mine[r * per_src:(r + 1) * per_src] = _ll_words(parts[r], epoch)
        before = resid.clone()
        out = arn.reduce_norm(i, resid, w, 1e-5)
        torch.cuda.synchronize()
        want_resid, want = _want(parts, before, w, 1e-5, dtype)
        assert arn.status() == 0
        assert torch.equal(resid, want_resid)
        assert ((out.float() - want).abs() <= ulp * want.abs() + 1e-6).all()
        for r in range(1, world):                                        # what this rank pushed into peer r's region
            got = recv[i][r].view(torch.int32)[0:per_src]
            assert torch.equal(got, _ll_words(parts[0], epoch))
        assert int(arn.sync[0]) == epoch and int(arn.sync[1]) == 0


def test_push_protocol_missing_peer_times_out_and_recovers(cuda_device):
    rows, hidden, dtype, world = 4, 1024, torch.bfloat16, 2
    g = torch.Generator().manual_seed(4)
    region = world * rows * hidden * 4
    recv = [[torch.zeros(region, dtype=torch.uint8, device=cuda_device) for _ in range(world)] for _ in range(2)]
    arn = glue.AllReduceNorm(rows, hidden, dtype, cuda_device, push_peers=recv, rank=0, max_spins=500, protocol="push")
    w = torch.ones(hidden, dtype=dtype, device=cuda_device)
    resid = torch.randn(rows, hidden, generator=g).to(dtype).to(cuda_device)
    parts = [(torch.randn(rows, hidden, generator=g) * 0.5).to(dtype).to(cuda_device) for _ in range(world)]
    before = resid.clone()
    arn.partial(0).copy_(parts[0])
    arn.reduce_norm(0, resid, w, 1e-5)                       # nothing has arrived from peer 1
    torch.cuda.synchronize()
    assert arn.status() == 1 and torch.equal(resid, before) and int(arn.sync[0]) == 1
    arn.sync[2] = 0
    arn.partial(1).copy_(parts[0])
    per_src = rows * hidden
    recv[1][0].view(torch.int32)[per_src:2 * per_src] = _ll_words(parts[1], 2)
    out = arn.reduce_norm(1, resid, w, 1e-5)
    torch.cuda.synchronize()
    want_resid, want = _want(parts, before, w, 1e-5, dtype)
    assert arn.status() == 0 and torch.equal(resid, want_resid)
    assert ((out.float() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-6).all()
