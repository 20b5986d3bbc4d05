"""Tensor-parallel collectives as our own NVLink kernels (no NCCL on the layer path).

For the 32-64 MB messages of sequence-parallel TP on two ranks NCCL picks its low-latency ring protocol and
moves ~120 GB/s; plain peer-to-peer loads and stores over NVSwitch move the same bytes several times faster.

* all-gather -> GEMM (column-parallel linears, and the gather of ``dY`` in the backward of row-parallel ones) is ONE
  kernel: :meth:`P2PComm.gemm_all_gather` launches the tcgen05 GEMM whose extra warps store this rank's rows into
  every rank's gathered buffer and signal, while its tiles of the own rows already run; tiles of a peer's rows start
  when that peer's flag has arrived (``ops/csrc/gemm_sm100.cu``, the ``AG`` variant).
* GEMM -> reduce-scatter (row-parallel linears, and the input gradient of column-parallel ones) is the GEMM whose
  epilogue TMA-stores each tile into its owner's memory, followed by a local sum (:meth:`P2PComm.gemm_reduce_scatter`).
* the remaining collectives (vision features, non-GEMM gathers) are: copy the contribution into a slot of this rank's
  symmetric staging buffer → ``signal`` (store the collective's sequence number into every peer's flag array,
  release/system scope) → one pull kernel that waits (bounded) for all signals and then reads the peers' slots
  directly (``ops/csrc/comm_kernels.cu``).  The reduce-scatter kernel accumulates in fp32 and can add a residual in
  the same pass.

Collectives are numbered 1, 2, ... in program order (identical on every rank, all on the caller's stream), and flag
values only grow, so "flag[r] >= e" means rank r has contributed to collective e.  Gathered activations that are kept
for backward live in one symmetric buffer per call site (``site_buffer``); a peer overwrites it in the next
micro-batch's forward, which :meth:`P2PComm.begin_microbatch` orders behind this rank's previous backward.

A waiting kernel gives up after a bounded time (``VLMT_FLAG_WAIT_MS``, default 20 s) and writes a status word (read by ``ops.cuda.check_status``)
instead of spinning forever, so a rank that left shows up as a Python exception on the survivors.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import symm


class P2PComm:
    N_SLOTS = 4

    FENCE_ROW = 16  # flags[16 + r]: micro-batch fence of rank r; flags[r]: collective number of rank r

    def __init__(self, group, device, slot_elems: int = 1 << 25):
        self.group, self.device = group, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.epoch = 0
        self.fence_epoch = 0
        self.slot_elems = 0
        self.staging = None
        self.flags = symm.symmetric_zeros(64, torch.int32, device, group)
        self.flag_ptrs = symm.peer_ptrs(self.flags)
        self.side = torch.cuda.Stream(device=device)  # pulls that overlap the caller's compute
        self.ag_counter = torch.zeros(1, dtype=torch.int32, device=device)  # CTAs done with their share of a push
        self.arena = symm.SymmetricArena(group, device)
        self.sites = {}  # call site -> (gathered buffer, its address on every rank)
        symm.apply_flag_wait_limit()
        self._alloc(slot_elems)

    def _alloc(self, slot_elems: int):
        """(Re)allocate the staging ring.  Peers may still be reading the old ring or storing into it, so every rank first
        drains its own stream and meets the others; only then is the old buffer dropped."""
        slot_elems = (slot_elems + 1023) // 1024 * 1024
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        old = self.staging
        self.staging = symm.symmetric_zeros(self.N_SLOTS * slot_elems, torch.bfloat16, self.device, self.group)
        self.slot_elems = slot_elems
        self.staging_ptrs = symm.peer_ptrs(self.staging)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # every rank's buffers are zeroed and mapped before the first signal
        if old is not None:
            symm.release(old)

    def reserve(self, n: int):
        """Make every staging slot hold at least ``n`` elements now (at set-up, from the model's sizes), so that no
        collective of the training loop has to grow the ring, which costs a device synchronisation and a barrier."""
        if n > self.slot_elems:
            self._alloc(n)

    def _slot(self, n: int):
        if n > self.slot_elems:
            self._alloc(n)
        self.epoch += 1
        s = self.epoch % self.N_SLOTS
        off = s * self.slot_elems
        return self.epoch, self.staging[off:off + n], [p + off * 2 for p in self.staging_ptrs]

    def site_buffer(self, site, rows: int, width: int):
        """The gathered-activation buffer ``[rows, width]`` of one call site (a module), allocated on first use from the
        symmetric arena and reused by every later step.  All ranks reach their call sites in the same order."""
        ent = self.sites.get(id(site))
        if ent is None or ent[0].numel() < rows * width:
            ent = self.arena.alloc(rows * width)
            self.sites[id(site)] = ent
        buf, ptrs = ent
        return buf[: rows * width].view(rows, width), ptrs

    def begin_microbatch(self):
        """Order the peers' stores of the coming forward pass behind this rank's previous backward pass: every rank
        announces "my stream has reached the next micro-batch" and waits (bounded, on the device) for the others."""
        from ..ops import cuda as cu

        self.fence_epoch += 1
        cu._C.signal_peers_at(self.flag_ptrs, self.FENCE_ROW, self.rank, self.fence_epoch)
        cu._C.wait_flags(self.flags.data_ptr(), self.FENCE_ROW, self.world, self.fence_epoch, self.rank)
        cu._tick(2)

    def gemm_all_gather(self, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False, site=None):
        """``(all_gather_rows(x_local) @ op(w), all_gather_rows(x_local))`` in one kernel launch (``op(w)`` = ``w.T``, or
        ``w`` with ``b_mn``).  The gathered rows land in the call site's persistent buffer (``site``: kept for backward)
        or, without a site, in a slot of the staging ring (valid until three more collectives have been issued)."""
        from ..ops import cuda as cu

        x_local = x_local.contiguous()
        R, K = x_local.shape
        T = R * self.world
        if site is not None:
            x_full, ptrs = self.site_buffer(site, T, K)
            self.epoch += 1
            e = self.epoch
        else:
            e, slot, ptrs = self._slot(T * K)
            x_full = slot.view(T, K)
        n_out = w.shape[1] if b_mn else w.shape[0]
        y = x_local.new_empty((T, n_out))
        cu._C.gemm_ag(x_local, x_full, w, y, ptrs, self.flag_ptrs, 0, self.ag_counter, e, self.rank, b_mn)
        cu._tick()
        return y, x_full

    def gemm_ag_usable(self, x, w, b_mn: bool = False) -> bool:
        n_out = w.shape[1] if b_mn else w.shape[0]
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] % 128 == 0 and x.shape[1] % 8 == 0
                and n_out > 128 and n_out % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and self.world <= 8)

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import cuda as cu

        x = x.contiguous()
        n = x.numel()
        e, slot, ptrs = self._slot(n)
        slot.copy_(x.view(-1))
        cu._C.signal_peers(self.flag_ptrs, self.rank, e)
        out = x.new_empty((x.shape[0] * self.world,) + tuple(x.shape[1:]))
        cu._C.pull_gather(ptrs, out, n, self.flags.data_ptr(), e)
        cu._tick(2)
        return out

    def all_gather_rows_async(self, x: torch.Tensor):
        """Like :meth:`all_gather_rows`, but the pull runs on this object's side stream: returns ``(out, event)``; the
        caller's stream must wait for ``event`` before it reads rows other than its own (which it still holds in ``x``),
        and can compute on its own rows meanwhile."""
        from ..ops import cuda as cu

        x = x.contiguous()
        n = x.numel()
        e, slot, ptrs = self._slot(n)
        slot.copy_(x.view(-1))
        cu._C.signal_peers(self.flag_ptrs, self.rank, e)
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        out = x.new_empty((x.shape[0] * self.world,) + tuple(x.shape[1:]))
        out.record_stream(self.side)
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            cu._C.pull_gather(ptrs, out, n, self.flags.data_ptr(), e)
            done = torch.cuda.Event()
            done.record(self.side)
        cu._tick(2)
        return out, done

    def reduce_scatter_begin(self, rows_total: int, width: int):
        """Reduce-scatter in two halves around the caller's compute: returns ``(buf, finish)``.  The caller writes its
        ``[rows_total, width]`` partial result into ``buf`` (this rank's staging slot, so no extra copy), calls
        ``finish.signal()`` as soon as the row blocks of the OTHER ranks are written, goes on to write its own block (and
        to do unrelated work), and finally calls ``finish.result(residual)``."""
        n = rows_total * width
        e, slot, ptrs = self._slot(n)
        return slot.view(rows_total, width), _ReduceScatterHandle(self, e, ptrs, rows_total // self.world, width)

    def reduce_scatter_rows(self, y: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        from ..ops import cuda as cu

        y = y.contiguous()
        n = y.numel()
        assert y.shape[0] % self.world == 0
        e, slot, ptrs = self._slot(n)
        slot.copy_(y.view(-1))
        cu._C.signal_peers(self.flag_ptrs, self.rank, e)
        out = y.new_empty((y.shape[0] // self.world,) + tuple(y.shape[1:]))
        cu._C.pull_reduce(ptrs, out, residual.contiguous() if residual is not None else None, n // self.world, self.rank,
                          self.flags.data_ptr(), e)
        cu._tick(2)
        return out


    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None,
                            b_mn: bool = False) -> torch.Tensor:
        """``reduce_scatter_rows(x @ w.T)`` (``x @ w`` with ``b_mn``: the input gradient of a column-parallel linear, ``w``
        stored ``[out, in]``) with the collective fused into the GEMM: the tcgen05 GEMM's epilogue stores each
        output tile directly into the staging slot of the rank that owns those rows (peer stores over NVLink, overlapping
        the remaining tiles); after the signal round every rank sums the ``world`` partial blocks it received — local
        reads only — and adds ``residual`` in the same pass."""
        from ..ops import cuda as cu

        M, N = x.shape[0], (w.shape[1] if b_mn else w.shape[0])
        rows = M // self.world
        n = M * N
        e, _slot, ptrs = self._slot(n)
        block = rows * N * 2  # bytes of one [rows, N] partial block
        dst = [p + self.rank * block for p in ptrs]  # on rank o: block `my rank` of its slot
        cu._C.gemm_rs_push(x, w, dst, rows, b_mn)
        cu._C.signal_peers(self.flag_ptrs, self.rank, e)
        out = x.new_empty((rows, N))
        mine = ptrs[self.rank]
        local = [mine + (r - self.rank) * block for r in range(self.world)]  # kernel adds rank * block: block r of my slot
        cu._C.pull_reduce(local, out, residual.contiguous() if residual is not None else None, rows * N, self.rank,
                          self.flags.data_ptr(), e)
        cu._tick(3)
        return out

    def gemm_rs_usable(self, x, w) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and x.shape[0] % (128 * self.world) == 0 and w.shape[0] % 8 == 0 and x.shape[1] % 8 == 0)


class _ReduceScatterHandle:
    def __init__(self, comm: P2PComm, epoch: int, ptrs, rows: int, width: int):
        self.comm, self.epoch, self.ptrs, self.rows, self.width = comm, epoch, ptrs, rows, width

    def signal(self):
        from ..ops import cuda as cu

        cu._C.signal_peers(self.comm.flag_ptrs, self.comm.rank, self.epoch)

    def result(self, like: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        from ..ops import cuda as cu

        out = like.new_empty((self.rows, self.width))
        cu._C.pull_reduce(self.ptrs, out, residual.contiguous() if residual is not None else None, self.rows * self.width,
                          self.comm.rank, self.comm.flags.data_ptr(), self.epoch)
        cu._tick(2)
        return out


def usable(x: torch.Tensor, ctx) -> bool:
    return (getattr(ctx, "p2p", None) is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % (8 * ctx.size) == 0)
