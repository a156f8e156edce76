"""Decode-step glue around the attention call: fused residual add + RMSNorm and SiLU(gate) * up.

With a handful of rows per step the separate framework kernels (add, norm, slice, silu, mul) are launch-bound;
these two launches replace seven.  The reference runs Hugging Face's ``LlamaRMSNorm`` / ``LlamaMLP`` modules
here (the model it patches, benchmarks/llama_integration_benchmark.py:266-279).
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _C, _lib, _workspace


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


def skinny_gemm_supported(rows: int, K: int, N: int) -> bool:
    """Shapes the weight-streaming GEMM serves: at most 16 rows, K a multiple of 32, N a multiple of 64."""
    return 0 < rows <= 16 and K % 32 == 0 and N % 64 == 0


def skinny_gemm(x: Tensor, w: Tensor, out: Tensor | None = None) -> Tensor:
    """``x [rows <= 16, K] @ w [K, N]`` (fp16 or bf16, fp32 accumulation) by the weight-streaming kernel.

    The decode step's projections: with a batch of 16 rows they are pure weight streaming, which this kernel does
    with every CTA reading an equal share of ``w`` (``skv_skinny_gemm``).  ``out`` may be any contiguous ``[rows, N]``
    tensor of the same dtype, for example the symmetric-memory buffer a fused all-reduce reads.
    """
    _check_2d(x, "x")
    _check_2d(w, "w")
    rows, K = x.shape
    N = w.shape[1]
    _C._require(w.shape[0] == K and w.dtype == x.dtype and w.device == x.device, "w must be [K, N] of x's dtype on x's device")
    _C._require(skinny_gemm_supported(rows, K, N), "skinny_gemm serves rows <= 16, K % 32 == 0, N % 64 == 0")
    if out is None:
        out = torch.empty((rows, N), dtype=x.dtype, device=x.device)
    else:
        _C._require(out.shape == (rows, N) and out.dtype == x.dtype and out.is_contiguous() and out.device == x.device,
                    "out must be a contiguous [rows, N] tensor of x's dtype on x's device")
    lib = _lib.load()
    dev = _C._dev_index(x)
    ws = _workspace.get("skinny_gemm", lib.skv_skinny_gemm_workspace_bytes(rows, K, N, dev), x.device)
    rc = lib.skv_skinny_gemm(x.data_ptr(), w.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), rows, K, N,
                             int(x.dtype == torch.bfloat16), dev, torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "skinny_gemm")
    return out


class AllReduceNorm:
    """Sum all-reduce over the GPUs of one node fused with the residual add and RMSNorm that consume it.

    Each rank's GEMM writes its partial ``[rows, hidden]`` result into ``partial(i)`` (``i`` alternates 0, 1
    between consecutive calls), a buffer in symmetric memory that every peer can read; ``reduce_norm(i, ...)``
    is then ONE kernel (``skv_allreduce_residual_rmsnorm``) that signals the peers, waits for them with a bounded
    spin, sums the partials over NVLink in rank order, adds the residual stream in place and returns the
    normalised rows.  No library collective runs; a wait that runs out is reported by :meth:`status`.
    ``peers`` (tests only) replaces the symmetric-memory rendezvous by explicit ``(partial, flags)`` tensors.
    """

    FLAG_WORDS = 8

    def __init__(self, rows: int, hidden: int, dtype: torch.dtype, device, group=None, *, max_spins: int = 1 << 21,
                 peers=None, rank: int | None = None, protocol: str = "pull", push_peers=None):
        """``protocol="push"``: every rank writes its partial, tagged with the call's epoch word by word, into the peers'
        receive regions and then polls its own (one NVLink traversal instead of a flag followed by remote loads;
        ``skv_allreduce_residual_rmsnorm_push``, rows of up to 4096 elements).  ``push_peers`` (tests only):
        ``push_peers[parity][r]`` = rank r's receive region, uint8 ``[world * rows * hidden * 4]``."""
        import ctypes

        _C._require(dtype in (torch.float16, torch.bfloat16), "dtype must be fp16 or bf16")
        _C._require(protocol in ("pull", "push"), "protocol must be 'pull' or 'push'")
        self.rows, self.hidden, self.dtype, self.device = rows, hidden, dtype, torch.device(device)
        self.max_spins = int(max_spins)
        self.protocol = protocol
        part_bytes = (rows * hidden * 2 + 255) // 256 * 256
        self.sync = torch.zeros(4, dtype=torch.int32, device=self.device)
        if protocol == "push":
            _C._require(hidden <= 4096, "the push protocol serves rows of up to 4096 elements")
            arr_t = None
            if push_peers is None:
                import torch.distributed as dist
                import torch.distributed._symmetric_memory as symm

                group = group if group is not None else dist.group.WORLD
                self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
                region = self.world * rows * hidden * 4
                self._buf = symm.empty(2 * region, dtype=torch.uint8, device=self.device)
                self._buf.zero_()
                torch.cuda.synchronize(self.device)
                handle = symm.rendezvous(self._buf, group)
                dist.barrier(group)                  # every rank's receive regions are zero before anybody pushes
                bases = [int(p) for p in handle.buffer_ptrs]
                recv_ptrs = [[b + i * region for b in bases] for i in range(2)]
            else:
                self.world, self.rank = len(push_peers[0]), int(rank or 0)
                self._keep = push_peers
                recv_ptrs = [[t.data_ptr() for t in push_peers[i]] for i in range(2)]
            self._partials = [torch.zeros((rows, hidden), dtype=dtype, device=self.device) for _ in range(2)]
            arr = ctypes.c_void_p * self.world
            self._recv_arr = [arr(*ptrs) for ptrs in recv_ptrs]
            return
        if peers is None:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm

            group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            self._buf = symm.empty(2 * part_bytes + 256, dtype=torch.uint8, device=self.device)
            self._buf.zero_()
            torch.cuda.synchronize(self.device)
            handle = symm.rendezvous(self._buf, group)
            dist.barrier(group)                      # every rank's flags are zero before anybody signals
            bases = [int(p) for p in handle.buffer_ptrs]
            self._partials = [self._buf[i * part_bytes:i * part_bytes + rows * hidden * 2].view(dtype).view(rows, hidden)
                              for i in range(2)]
            part_ptrs = [[b + i * part_bytes for b in bases] for i in range(2)]
            flag_ptrs = [b + 2 * part_bytes for b in bases]
        else:
            self.world, self.rank = len(peers[0]), int(rank or 0)
            self._keep = peers
            self._partials = [peers[i][self.rank][0] for i in range(2)]
            part_ptrs = [[p[0].data_ptr() for p in peers[i]] for i in range(2)]
            flag_ptrs = [p[1].data_ptr() for p in peers[0]]
        arr = ctypes.c_void_p * self.world
        self._part_arr = [arr(*ptrs) for ptrs in part_ptrs]
        self._flag_arr = arr(*flag_ptrs)

    def partial(self, i: int) -> Tensor:
        """This rank's partial-sum buffer ``i`` (0 or 1): pass it as ``out=`` of the GEMM that produces the partial."""
        return self._partials[i]

    def reduce_norm(self, i: int, resid: Tensor, weight: Tensor, eps: float, out: Tensor | None = None) -> Tensor:
        _check_2d(resid, "resid")
        _C._require(resid.shape == (self.rows, self.hidden) and resid.dtype == self.dtype, "resid must match the buffers")
        _C._require(weight.shape == (self.hidden,) and weight.dtype == self.dtype and weight.is_contiguous(),
                    "weight must be a contiguous [hidden] vector of the buffers' dtype")
        if out is None:
            out = torch.empty_like(resid)
        if self.protocol == "push":
            rc = _lib.load().skv_allreduce_residual_rmsnorm_push(
                self._partials[i].data_ptr(), self._recv_arr[i], self.sync.data_ptr(), resid.data_ptr(), weight.data_ptr(),
                out.data_ptr(), self.rows, self.hidden, float(eps), int(self.dtype == torch.bfloat16), self.rank, self.world,
                self.max_spins, _C._dev_index(resid), torch.cuda.current_stream(resid.device).cuda_stream)
            _lib.check(rc, "allreduce_residual_rmsnorm_push")
            return out
        rc = _lib.load().skv_allreduce_residual_rmsnorm(
            self._part_arr[i], self._flag_arr, self.sync.data_ptr(), resid.data_ptr(), weight.data_ptr(), out.data_ptr(),
            self.rows, self.hidden, float(eps), int(self.dtype == torch.bfloat16), self.rank, self.world, self.max_spins,
            _C._dev_index(resid), torch.cuda.current_stream(resid.device).cuda_stream)
        _lib.check(rc, "allreduce_residual_rmsnorm")
        return out

    def status(self) -> int:
        """Device status word (synchronises): 0, or 1 when a peer did not arrive within ``max_spins`` polls."""
        return int(self.sync[2].item())
