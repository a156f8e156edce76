"""Records outputs of the REFERENCE's own CUDA kernels (rebuilt for sm_100a) as golden fixtures.

Needs a GPU and the module built by ``oracle/build_ref.py`` (the reference's three ``.cu`` files
and its pybind file compiled unchanged).  Run from the repository root:

    python tests/golden/make_refcuda_golden.py [output.npz]

and commit the result as ``tests/golden/refcuda_outputs.npz``.  Inputs are regenerated from seeds
by the tests; the fixture stores a SHA-256 of them beside every output.  What is recorded:

  * ``sparse_attention_forward`` (csrc/kernels/sparse_attention.cu:178-244): the block-mean rule at
    config 1's block path (T=1024, D=64, 64x4), at T=300 (ragged last block), at T=300 with more
    blocks asked for than exist, and at T=4096, H=32, D=128, 64x8;
  * ``fused_gqa`` (csrc/kernels/gqa_decode.cu:218-290) at N=4096 and a ragged N=5000;
  * ``kv_evict_quant_forward`` (csrc/kernels/kv_evict_quant.cu:272-364) at the shape of the
    reference's GPU test (tests/test_kernel_correctness.py:5): its top-k is approximate, so the
    tests compare it only with the reference's own loose bound.

Each kernel is scalar CUDA C without waits; shapes are kept below 2^31 elements because the
kernels index with 32-bit integers.
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from llm_inference_optimization_b200 import workloads  # noqa: E402
from oracle import build_ref  # noqa: E402


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().cpu().numpy().tobytes())
    return h.hexdigest()


def block_inputs(name: str):
    """fp16 Q [B,H,1,D], K/V [B,H,T,D] of the named block-sparse case (CPU, seeded)."""
    if name == "config1":
        return tuple(t.half() for t in workloads.token_sparse_config1())
    if name == "ragged300":
        torch.manual_seed(21)
        return torch.randn(1, 8, 1, 64).half(), torch.randn(1, 8, 300, 64).half(), torch.randn(1, 8, 300, 64).half()
    if name == "ctx4096":
        torch.manual_seed(22)
        return (torch.randn(1, 32, 1, 128).half(), torch.randn(1, 32, 4096, 128).half(),
                torch.randn(1, 32, 4096, 128).half())
    raise KeyError(name)


BLOCK_CASES = [("config1", 64, 4), ("ragged300", 64, 4), ("ragged300", 64, 8), ("ctx4096", 64, 8)]
DENSE_CASES = [4096, 5000]


def token_inputs():
    """The reference GPU test's shape: B,H,N,D = 1,32,4096,128 (seed 42), fp16."""
    torch.manual_seed(42)
    return (torch.randn(1, 32, 1, 128).half(), torch.randn(1, 32, 4096, 128).half(),
            torch.randn(1, 32, 4096, 128).half())


def main(out_path: Path) -> None:
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    ref = build_ref.load()
    dev = torch.device("cuda", 0)
    rec = {}
    for name, bs, k in BLOCK_CASES:
        Q, K, V = block_inputs(name)
        out = ref.sparse_attention_forward(Q.to(dev), K.to(dev).contiguous(), V.to(dev).contiguous(), bs, k)
        torch.cuda.synchronize()
        rec[f"block_{name}_bs{bs}_k{k}"] = out.cpu().numpy()
        rec[f"block_{name}_sha256"] = np.array(digest(Q, K, V))
    for n in DENSE_CASES:
        Q, K, V, scale = workloads.dense_gqa(n)
        out = ref.fused_gqa(Q.to(dev), K.to(dev), V.to(dev), scale)
        torch.cuda.synchronize()
        rec[f"dense_n{n}"] = out.cpu().numpy()
        rec[f"dense_n{n}_sha256"] = np.array(digest(Q, K, V))
    Q, K, V = token_inputs()
    out = ref.kv_evict_quant_forward(Q.to(dev), K.to(dev), V.to(dev), 32, False)
    torch.cuda.synchronize()
    rec["token_k32"] = out.cpu().numpy()
    rec["token_sha256"] = np.array(digest(Q, K, V))
    rec["device"] = np.array(torch.cuda.get_device_name(0))
    rec["torch"] = np.array(torch.__version__)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, sorted(rec))


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent / "refcuda_outputs.npz")
