"""Decode-step glue around the attention call: fused residual add + RMSNorm and SiLU(gate) * up.

With a handful of rows per step the separate framework kernels (add, norm, slice, silu, mul) are launch-bound;
these two launches replace seven.  The reference runs Hugging Face's ``LlamaRMSNorm`` / ``LlamaMLP`` modules
here (the model it patches, benchmarks/llama_integration_benchmark.py:266-279).
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _C, _lib


def _check_2d(t: Tensor, what: str) -> None:
    _C._require(t.is_cuda and t.dim() == 2 and t.is_contiguous() and t.dtype in (torch.float16, torch.bfloat16),
                f"{what} must be a contiguous fp16 or bf16 CUDA matrix")


def residual_rmsnorm(resid: Tensor, delta: Tensor | None, weight: Tensor, eps: float, out: Tensor | None = None) -> Tensor:
    """``resid += delta`` in place (when ``delta`` is given), then return ``rms_norm(resid) * weight``.

    ``resid``, ``delta`` ``[rows, hidden]`` and ``weight`` ``[hidden]`` share one dtype (fp16 or bf16).
    """
    _check_2d(resid, "resid")
    rows, hidden = resid.shape
    if delta is not None:
        _check_2d(delta, "delta")
        _C._require(delta.shape == resid.shape and delta.dtype == resid.dtype and delta.device == resid.device,
                    "delta must match resid")
    _C._require(weight.shape == (hidden,) and weight.dtype == resid.dtype and weight.is_contiguous()
                and weight.device == resid.device, "weight must be a contiguous [hidden] vector of resid's dtype")
    if out is None:
        out = torch.empty_like(resid)
    rc = _lib.load().skv_residual_rmsnorm(
        None if delta is None else delta.data_ptr(), resid.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, hidden,
        float(eps), int(resid.dtype == torch.bfloat16), _C._dev_index(resid),
        torch.cuda.current_stream(resid.device).cuda_stream)
    _lib.check(rc, "residual_rmsnorm")
    return out


def silu_mul(gate_up: Tensor, out: Tensor | None = None) -> Tensor:
    """``silu(gate_up[:, :I]) * gate_up[:, I:]`` for ``gate_up [rows, 2*I]`` (fp16 or bf16), one launch."""
    _check_2d(gate_up, "gate_up")
    rows, two_i = gate_up.shape
    _C._require(two_i % 16 == 0, "gate_up must have an even number of 8-element groups per row")
    inter = two_i // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    rc = _lib.load().skv_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, inter, int(gate_up.dtype == torch.bfloat16),
                                  _C._dev_index(gate_up), torch.cuda.current_stream(gate_up.device).cuda_stream)
    _lib.check(rc, "silu_mul")
    return out
