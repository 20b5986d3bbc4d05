"""Symmetric (peer-visible) device memory.

Buffers come from torch's symmetric-memory allocator (CUDA VMM allocations whose handles are
exchanged over the process-group store), which maps every rank's buffer into every other
rank's address space and, where the fabric supports it, binds them to an NVLS multicast
object.  Kernels only ever see raw pointers: ``peer_ptrs(t)`` (one per rank) and
``multicast_ptr(t)`` (0 when unavailable).  Setting ``VLMT_NO_MULTIMEM=1`` forces the plain
peer-pointer path (used by failure-handling tests, where a rank may leave while mapped).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

_HANDLES: dict[int, object] = {}


def available(device) -> bool:
    return torch.device(device).type == "cuda" and dist.is_initialized()


def symmetric_zeros(n: int, dtype, device, group) -> torch.Tensor:
    import torch.distributed._symmetric_memory as symm_mem

    t = symm_mem.empty(n, dtype=dtype, device=device)
    t.zero_()
    grp = group if group is not None else dist.group.WORLD
    hdl = symm_mem.rendezvous(t, group=grp)
    _HANDLES[t.data_ptr()] = hdl
    return t


def handle_of(t: torch.Tensor):
    return _HANDLES.get(t.untyped_storage().data_ptr()) or _HANDLES.get(t.data_ptr())


def peer_ptrs(t: torch.Tensor) -> list[int]:
    """Device addresses of this buffer on every rank of its group (own rank included)."""
    return [int(p) for p in handle_of(t).buffer_ptrs]


def multicast_ptr(t: torch.Tensor) -> int:
    if os.environ.get("VLMT_NO_MULTIMEM", "0") == "1":
        return 0
    hdl = handle_of(t)
    try:
        return int(hdl.multicast_ptr) if hdl.has_multicast_support(hdl.device.type if hasattr(hdl, "device") else "cuda", hdl.device.index) else 0
    except Exception:
        try:
            return int(hdl.multicast_ptr)
        except Exception:
            return 0


def apply_flag_wait_limit():
    """Set the bound of the in-kernel flag waits of the current device from ``VLMT_FLAG_WAIT_MS`` (default 20 000)."""
    from ..ops import cuda as cu

    cu._C.set_flag_wait_ms(int(os.environ.get("VLMT_FLAG_WAIT_MS", "20000")))
