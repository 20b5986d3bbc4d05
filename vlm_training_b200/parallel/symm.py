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


def release(t: torch.Tensor):
    """Forget the rendezvous handle of a symmetric buffer that is no longer used (the mapping goes away with the last
    reference to the tensor and its handle)."""
    _HANDLES.pop(t.data_ptr(), None)


class SymmetricArena:
    """Bump allocator over symmetric memory for buffers that live as long as the model (one per call site that
    gathers activations).  Every rank of the group must request the same sizes in the same order, so a buffer has the
    same offset on every rank; memory comes in chunks so that ~70 call sites cost a handful of rendezvous, not 70."""

    def __init__(self, group, device, chunk_bytes: int = 1 << 30):
        self.group, self.device, self.chunk_bytes = group, device, chunk_bytes
        self.chunks = []  # (uint8 tensor, peer pointers, bytes used)

    def alloc(self, n: int, dtype=torch.bfloat16):
        """Returns ``(tensor [n], [address of the same buffer on every rank])``; the buffer is zero-filled."""
        nbytes = (n * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        if not self.chunks or self.chunks[-1][2] + nbytes > self.chunks[-1][0].numel():
            size = max(self.chunk_bytes, nbytes)
            buf = symmetric_zeros(size, torch.uint8, self.device, self.group)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # zero-filled and mapped on every rank before anybody stores into it
            self.chunks.append([buf, peer_ptrs(buf), 0])
        buf, ptrs, used = self.chunks[-1]
        self.chunks[-1][2] = used + nbytes
        t = buf[used:used + n * torch.empty((), dtype=dtype).element_size()].view(dtype)
        return t, [p + used for p in ptrs]

    def bytes_reserved(self) -> int:
        return sum(c[0].numel() for c in self.chunks)


def apply_flag_wait_limit():
    """Set the bound of the in-kernel flag waits of the current device from ``VLMT_FLAG_WAIT_MS`` (default 20 000)."""
    from ..ops import cuda as cu

    ms = int(os.environ.get("VLMT_FLAG_WAIT_MS", "20000"))
    cu._C.set_flag_wait_ms(ms)
    cu._C.gemm_set_flag_wait_ms(ms)
