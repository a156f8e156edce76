"""Per-(device, stream) scratch buffers handed to the C-ABI as workspaces.

The kernels keep a status word and atomic tickets in their workspace and leave
both zero when they finish, so a buffer is zero-filled once, when it is first
allocated or grown, and then reused by every later call on the same stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_cache: dict[tuple[str, int, int], torch.Tensor] = {}


def get(kind: str, nbytes: int, device: torch.device) -> torch.Tensor:
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (kind, device.index if device.index is not None else torch.cuda.current_device(), stream)
    buf = _cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 4096), dtype=torch.uint8, device=device)
        _cache[key] = buf
    return buf


def all_of(kind: str, device: torch.device) -> list[torch.Tensor]:
    """Every cached workspace of one kind on a device (one per stream that has launched with it)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    return [buf for (k, d, _), buf in _cache.items() if k == kind and d == index]


def status(buf: torch.Tensor) -> int:
    """Read (and synchronise on) the device status word of a workspace."""
    out = C.c_int(0)
    dev = buf.device.index
    st = torch.cuda.current_stream(buf.device).cuda_stream
    _lib.check(_lib.load().skv_workspace_status(buf.data_ptr(), dev, st, C.byref(out)), "skv_workspace_status")
    return out.value


def clear() -> None:
    _cache.clear()
