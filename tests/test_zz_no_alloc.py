"""The allocation-free dense-decode entry point gives the same output as the workspace one.

Some hosts of this library cannot allocate device memory when they decode: an inference server that
has given all free HBM to its KV page pool, or a non-torch host with no caching allocator to lend a
workspace.  ``skv_gqa_decode_noalloc`` serves them from a fixed 4 MiB array inside the library.
This file is collected last on purpose, so a failure here cannot hide another test's result.
"""
import pytest
import torch

from llm_inference_optimization_b200 import _C, _lib, workloads

pytestmark = pytest.mark.gpu
TOL = 2e-3  # the max-abs bound used by the dense-decode parity tests


def call_noalloc(lib, Q, K, V, scale, out, seq_lens=None):
    B, Hq, D = Q.shape
    N, Hkv = K.shape[1], K.shape[2]
    dev = Q.device.index
    rc = lib.skv_gqa_decode_noalloc(
        Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), B, N, Hq, Hkv, D,
        K.stride(0), K.stride(1), K.stride(2), None if seq_lens is None else seq_lens.data_ptr(),
        float(scale), dev, torch.cuda.current_stream(Q.device).cuda_stream)
    _lib.check(rc, "skv_gqa_decode_noalloc")


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row(cuda_device, lib):
    # two different problems back to back: the second call finds the first call's partials in the array
    for N, B, seed in ((20000, 1, 31), (3001, 2, 32)):
        Q, K, V, scale = workloads.dense_gqa(N, B=B, seed=seed)
        Qd, Kd, Vd = Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device)
        want = _C.fused_gqa(Qd, Kd, Vd, scale)          # existing entry point, torch-allocated workspace
        got = torch.full_like(want, float("nan"))       # caller-provided output, pre-poisoned
        before = torch.cuda.memory_allocated(cuda_device)
        call_noalloc(lib, Qd, Kd, Vd, scale, got)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(cuda_device) == before
        assert not torch.isnan(got).any()
        assert (got.float() - want.float()).abs().max().item() <= TOL


def test_noalloc_entry_rejects_problems_beyond_its_scratch(cuda_device, lib):
    B, Hq, Hkv, D, N = 256, 64, 64, 128, 64  # B*Hq*D*4 bytes of partials alone exceed 4 MiB
    assert lib.skv_gqa_decode_workspace_bytes(B, N, Hq, Hkv, D, 0) > (4 << 20)
    Q = torch.zeros(B, Hq, D, dtype=torch.float16, device=cuda_device)
    K = torch.zeros(B, N, Hkv, D, dtype=torch.float16, device=cuda_device)
    out = torch.empty_like(Q)
    with pytest.raises(RuntimeError, match="scratch"):
        call_noalloc(lib, Q, K, K, 1.0, out)


def test_noalloc_status_word_is_readable_and_clean(cuda_device, lib):
    """The built-in array's status word can be read back (a caller of this entry never holds a workspace pointer)."""
    import ctypes
    Q, K, V, scale = workloads.dense_gqa(4096, seed=33)
    Qd, Kd, Vd = Q.to(cuda_device), K.to(cuda_device), V.to(cuda_device)
    out = torch.empty_like(Qd)
    call_noalloc(lib, Qd, Kd, Vd, scale, out)
    st = ctypes.c_int(-1)
    rc = lib.skv_gqa_decode_noalloc_status(cuda_device.index, torch.cuda.current_stream(cuda_device).cuda_stream, ctypes.byref(st))
    _lib.check(rc, "skv_gqa_decode_noalloc_status")
    assert st.value == 0
