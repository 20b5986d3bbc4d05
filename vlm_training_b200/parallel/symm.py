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
# Debug aid (VLMT_DEBUG_GUARDS=1): every symmetric buffer is allocated with a canary band in front of and behind the
# part that is handed out.  Peers reach these buffers by raw pointer arithmetic inside kernels, so a wrong offset or
# count on ANY rank shows up as a damaged band on the victim; `check_guards()` (called by the trainer after every step in
# this mode) names the buffer.  Bands cost 2 x 4 KiB per buffer and a device read per check; off by default.
GUARD_BYTES = 4096
_GUARD_PATTERN = 0x5A
_GUARDED: list = []  # (label, whole uint8 view, payload bytes)


def guards_enabled() -> bool:
    return os.environ.get("VLMT_DEBUG_GUARDS", "0") == "1"


def available(device) -> bool:
    return torch.device(device).type == "cuda" and dist.is_initialized()


def symmetric_zeros(n: int, dtype, device, group, label: str = "") -> torch.Tensor:
    import torch.distributed._symmetric_memory as symm_mem

    grp = group if group is not None else dist.group.WORLD
    if not guards_enabled():
        t = symm_mem.empty(n, dtype=dtype, device=device)
        t.zero_()
        hdl = symm_mem.rendezvous(t, group=grp)
        _HANDLES[t.data_ptr()] = hdl
        return t
    esz = torch.empty((), dtype=dtype).element_size()
    payload = (n * esz + 255) // 256 * 256
    raw = symm_mem.empty(payload + 2 * GUARD_BYTES, dtype=torch.uint8, device=device)
    raw.zero_()
    raw[:GUARD_BYTES].fill_(_GUARD_PATTERN)
    raw[GUARD_BYTES + payload:].fill_(_GUARD_PATTERN)
    hdl = symm_mem.rendezvous(raw, group=grp)
    t = raw[GUARD_BYTES:GUARD_BYTES + n * esz].view(dtype)
    _HANDLES[t.data_ptr()] = _OffsetHandle(hdl, GUARD_BYTES)
    _GUARDED.append((label or f"symmetric buffer of {n} x {dtype}", raw, payload))
    return t


class _OffsetHandle:
    """A rendezvous handle whose buffer addresses point behind the leading guard band."""

    def __init__(self, hdl, offset: int):
        self._hdl, self._offset = hdl, offset

    @property
    def buffer_ptrs(self):
        return [int(p) + self._offset for p in self._hdl.buffer_ptrs]

    @property
    def multicast_ptr(self):
        mc = int(self._hdl.multicast_ptr)
        return mc + self._offset if mc else 0

    def __getattr__(self, name):
        return getattr(self._hdl, name)


def check_guards():
    """Raise if a canary band of any guarded symmetric buffer on THIS rank has been written to (debug mode only)."""
    for label, raw, payload in _GUARDED:
        front = raw[:GUARD_BYTES]
        back = raw[GUARD_BYTES + payload:]
        bad_f = int((front != _GUARD_PATTERN).sum().item())
        bad_b = int((back != _GUARD_PATTERN).sum().item())
        if bad_f or bad_b:
            raise RuntimeError(f"out-of-bounds store into peer-visible memory: {label}: {bad_f} bytes damaged in front of the "
                               f"buffer, {bad_b} behind it")


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
