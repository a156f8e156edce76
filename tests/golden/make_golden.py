"""Generates the golden fixtures in this folder from the reference's own Python functions.

Run once, in a container where the reference checkout is mounted:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py <path to the reference checkout>

It imports ``sparse_kv.attention._reference_sparse_attention`` and
``sparse_kv.eviction._reference_eviction`` unmodified, evaluates them on seeded
CPU inputs and stores the results (plus small inputs, or a checksum of large
seeded ones) as ``.npz`` files.  The tests never need the reference checkout.
"""
import hashlib
import sys
import warnings
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def config1_inputs():
    """B=1, H=8, D=64, context 1024, one query token, N(0,1), seed 0 (fp32)."""
    torch.manual_seed(0)
    Q = torch.randn(1, 8, 1, 64)
    K = torch.randn(1, 8, 1024, 64)
    V = torch.randn(1, 8, 1024, 64)
    return Q, K, V


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from sparse_kv.attention import _reference_sparse_attention as ref_attn
        from sparse_kv.eviction import _reference_eviction as ref_evict

    # --- config 1, token-sparse path: fp32 inputs and the fp16-rounded inputs the CUDA path sees
    Q, K, V = config1_inputs()
    Qh, Kh, Vh = (t.half().float() for t in (Q, K, V))
    np.savez_compressed(
        HERE / "config1_token_sparse.npz",
        inputs_sha256=np.array(digest(Q, K, V)),
        out_k256_s0=ref_attn(Q, K, V, 256, 0).numpy(),
        out_k256_s4=ref_attn(Q, K, V, 256, 4).numpy(),
        out_k32_s4=ref_attn(Q, K, V, 32, 4).numpy(),
        out_h_k256_s0=ref_attn(Qh, Kh, Vh, 256, 0).numpy(),
        out_h_k256_s4=ref_attn(Qh, Kh, Vh, 256, 4).numpy(),
        out_h_k32_s4=ref_attn(Qh, Kh, Vh, 32, 4).numpy(),
    )

    # --- the shape family of the reference's own unit tests (16 query rows, context 512)
    torch.manual_seed(11)
    Q2, K2, V2 = torch.randn(1, 8, 16, 64), torch.randn(1, 8, 512, 64), torch.randn(1, 8, 512, 64)
    np.savez_compressed(
        HERE / "token_sparse_multiquery.npz",
        inputs_sha256=np.array(digest(Q2, K2, V2)),
        out_k64_s4=ref_attn(Q2, K2, V2, 64, 4).numpy(),
        out_h_k64_s4=ref_attn(Q2.half().float(), K2.half().float(), V2.half().float(), 64, 4).numpy(),
    )

    # --- eviction on a small cache, inputs stored
    torch.manual_seed(5)
    Ke, Ve = torch.randn(2, 3, 96, 16), torch.randn(2, 3, 96, 16)
    scores = torch.softmax(2.0 * torch.randn(2, 3, 4, 96), -1).sum(2)
    Ko, Vo = ref_evict(Ke, Ve, scores, 24, False)
    Ko8, Vo8 = ref_evict(Ke * 20, Ve * 20, scores, 24, True)
    np.savez_compressed(
        HERE / "eviction_small.npz",
        K=Ke.numpy(), V=Ve.numpy(), scores=scores.numpy(),
        topk_idx=scores.topk(24, dim=-1).indices.numpy(),
        K_out=Ko.numpy(), V_out=Vo.numpy(), K_out_cast_int8=Ko8.numpy(), V_out_cast_int8=Vo8.numpy(),
    )
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
