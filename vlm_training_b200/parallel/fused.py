"""One-kernel NVLink path of the sharded optimizer engine.

Per bucket, ``reduce_scatter(grads) → AdamW(shard) → all_gather(params)`` (three passes over HBM and two NCCL
kernels) becomes a single kernel that pulls the gradient shard from every peer (or one in-switch
``multimem.ld_reduce``), updates the fp32 state and pushes the bf16 parameters to every peer
(``ops/csrc/comm_kernels.cu``).  The engine's flat buffers live in symmetric memory for this.

The kernel for a bucket is launched from the autograd hook of the bucket's last gradient, so it overlaps the rest
of backward.  Ordering is by flags in symmetric memory, one row of ``world`` int32 per bucket, written with the
optimizer step number:

* when a rank has produced all gradients of bucket ``b`` it stores the step number into ``flag[b][rank]`` on every
  rank (``signal`` — on its own stream, so a signal never queues behind a wait);
* a rank's fused kernel for ``b`` is preceded by a one-block wait kernel that returns once ``flag[b][r] >= step`` for
  all OTHER ranks ``r`` (its own gradients are ordered by the stream; a kernel never waits for a separate launch on its
  own GPU): then every peer's gradients of ``b`` are final AND every peer is done reading the old parameters of ``b``;
* after its last bucket a rank signals row ``DONE``; before the next forward (and before gradients are cleared) every
  rank waits for all ``DONE`` signals: all pushes have landed and nobody still reads this step's gradients.

Every wait is bounded (``VLMT_FLAG_WAIT_MS``, default 20 s) and reports through the status word instead of hanging.

Gradient clipping needs the global norm before the first update, so with ``max_grad_norm`` the step is two kernels per
bucket: the reduce-scatter half runs from the gradient hooks as above (it keeps the reduced shard in fp32 and adds its
sum of squares to a device scalar), then one small all-reduce of that scalar, then the AdamW + all-gather half of every
bucket, which reads the clip factor from device memory — still no host read and no library collective on the buckets.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import symm


class FusedStepState:
    """Flags, streams and per-step bookkeeping of one engine."""

    def __init__(self, engine):
        self.engine = engine
        dev = engine.device
        self.signal_stream = torch.cuda.Stream(device=dev)
        symm.apply_flag_wait_limit()
        self.domains = []
        for d in engine.domains:
            info = {"domain": d, "flags": None}
            if d.size > 1:
                rows = len(d.buckets) + 1  # + DONE row
                d_flags = symm.symmetric_zeros(rows * d.size, torch.int32, dev, d.group)
                # the in-switch reduction pays once several peers would otherwise each send their copy of the shard; on two
                # ranks plain peer loads and stores measured 0.40 ms against 0.69 ms per 256 MB bucket
                use_mc = d.size >= 4 or os.environ.get("VLMT_FORCE_MULTIMEM", "0") == "1"
                info.update(flags=d_flags, flag_ptrs=symm.peer_ptrs(d_flags), done_row=len(d.buckets),
                            g_ptrs=symm.peer_ptrs(d.flat_grad), p_ptrs=symm.peer_ptrs(d.flat_param),
                            g_mc=symm.multicast_ptr(d.flat_grad) if use_mc else 0,
                            p_mc=symm.multicast_ptr(d.flat_param) if use_mc else 0)
            self.domains.append(info)
        torch.cuda.synchronize(dev)
        for d in engine.domains:
            if d.size > 1:
                dist.barrier(group=d.group)
        self.step = 0          # number of the optimizer step whose buckets are being processed
        self.processed = set()
        self.clip = engine.max_grad_norm is not None
        if self.clip:
            self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            for info in self.domains:
                d = info["domain"]
                info["red"] = [torch.empty(d.shard_range(b)[1] - d.shard_range(b)[0], dtype=torch.float32, device=dev) for b in d.buckets]

    def info_of(self, d):
        for info in self.domains:
            if info["domain"] is d:
                return info
        raise KeyError


def usable(engine) -> tuple[bool, str]:
    """Whether the one-kernel path can run this engine, and if not, why (the engine logs the reason and takes the
    NCCL path)."""
    for d in engine.domains:
        if d.exp_avg and d.exp_avg[0].dtype not in (torch.float32, torch.bfloat16):
            return False, f"the fused kernel keeps fp32 or bf16 Adam moments, optimizer_state_dtype is {d.exp_avg[0].dtype}"
        if d.size > 1 and symm.handle_of(d.flat_grad) is None:
            return False, f"the buffers of domain '{d.name}' are not in symmetric memory"
    return True, ""


def begin_step(engine):
    st: FusedStepState = engine._fused
    if st.step != engine.step_count + 1:
        st.step = engine.step_count + 1
        st.processed = set()


def process_bucket(engine, d, bi: int):
    """Signal 'my gradients of bucket bi are final', then (after every rank's signal) run the fused kernel on it."""
    from ..ops import cuda as cu

    st: FusedStepState = engine._fused
    begin_step(engine)
    key = (id(d), bi)
    if key in st.processed:
        return
    st.processed.add(key)
    info = st.info_of(d)
    b = d.buckets[bi]
    b.reduced = True
    step = st.step
    b1, b2 = engine.betas
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    if engine._identical and d.name == "tp_replicated":
        for p in b.params:
            if getattr(p, "_tp_grad", "partial") == "identical":
                p.grad.mul_(engine._identical_scale)
    cur = torch.cuda.current_stream()
    ev = torch.cuda.Event()
    ev.record(cur)
    world = d.size
    if world > 1:
        with torch.cuda.stream(st.signal_stream):
            st.signal_stream.wait_event(ev)
            cu._C.signal_peers_at(info["flag_ptrs"], bi * world, d.rank, step)
    esz = d.flat_grad.element_size()
    with torch.cuda.stream(engine.comm_stream):
        engine.comm_stream.wait_event(ev)
        if world > 1:
            cu._C.wait_flags(info["flags"].data_ptr(), bi * world, world, step, d.rank)  # own readiness: stream order
            g_ptrs, p_ptrs, g_mc, p_mc = info["g_ptrs"], info["p_ptrs"], info["g_mc"], info["p_mc"]
        else:
            g_ptrs, p_ptrs, g_mc, p_mc = [d.flat_grad.data_ptr()], [d.flat_param.data_ptr()], 0, 0
        lo, hi = d.shard_range(b)
        if st.clip:
            # first half only: the reduced shard (fp32) and its sum of squares; the update follows in finish_step
            cu._C.rs_reduce_sumsq([p + b.start * esz for p in g_ptrs], (g_mc + b.start * esz) if g_mc else 0, lo - b.start, hi - b.start,
                                  info["red"][bi], 0, st.sumsq)
            cu._tick()
            return
        _update_segments(engine, d, bi, g_ptrs, p_ptrs, g_mc, p_mc, world)


def _update_segments(engine, d, bi, g_ptrs, p_ptrs, g_mc, p_mc, world, red=None, sumsq=None):
    """AdamW (+ all-gather) on this rank's shard of bucket ``bi``, one launch per learning-rate group segment."""
    from ..ops import cuda as cu

    st: FusedStepState = engine._fused
    b = d.buckets[bi]
    esz = d.flat_grad.element_size()
    step = st.step
    b1, b2 = engine.betas
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    lo, hi = d.shard_range(b)
    for seg in b.segments:
        s, e = max(seg.start, lo), min(seg.end, hi)
        if e <= s:
            continue
        # parameters start on 8-element boundaries; a segment's tail may not end on one: the padding behind it
        # holds zero gradients, so rounding the end up is harmless
        e = min(hi, (e + 7) // 8 * 8)
        pg = engine.param_groups[seg.group]
        if red is not None:
            cu._C.adamw_push(red, s - lo, sumsq, float(engine.max_grad_norm), [p + b.start * esz for p in p_ptrs],
                             (p_mc + b.start * esz) if p_mc else 0, s - b.start, e - b.start, d.master[bi], d.exp_avg[bi],
                             d.exp_avg_sq[bi], s - lo, pg["lr"], b1, b2, engine.eps, pg["weight_decay"], bc1, bc2, d.grad_scale)
        else:
            cu._C.fused_rs_adamw_ag(
                [p + b.start * esz for p in g_ptrs], [p + b.start * esz for p in p_ptrs],
                (g_mc + b.start * esz) if g_mc else 0, (p_mc + b.start * esz) if p_mc else 0,
                world, s - b.start, e - b.start, d.master[bi], d.exp_avg[bi], d.exp_avg_sq[bi], s - lo,
                pg["lr"], b1, b2, engine.eps, pg["weight_decay"], bc1, bc2, d.grad_scale, world == 1)
        cu._tick()


def finish_step(engine):
    """Process whatever the hooks did not reach, then the DONE round; returns with the current stream ordered after it."""
    from ..ops import cuda as cu

    st: FusedStepState = engine._fused
    begin_step(engine)
    for d in engine.domains:
        for bi in range(len(d.buckets)):
            process_bucket(engine, d, bi)
    step = st.step
    with torch.cuda.stream(engine.comm_stream):
        if st.clip:
            # every rank's shards are disjoint: the global sum of squares is one all-reduce of a scalar, then the update
            if dist.is_initialized():
                dist.all_reduce(st.sumsq)
            for info in st.domains:
                d = info["domain"]
                for bi in range(len(d.buckets)):
                    if d.size > 1:
                        _update_segments(engine, d, bi, None, info["p_ptrs"], 0, info["p_mc"], d.size, info["red"][bi], st.sumsq)
                    else:
                        _update_segments(engine, d, bi, None, [d.flat_param.data_ptr()], 0, 0, 1, info["red"][bi], st.sumsq)
            engine.last_grad_norm = st.sumsq.sqrt() * engine.domains[0].grad_scale   # a device tensor: no host read here
            st.sumsq = torch.zeros_like(st.sumsq)
        for info in st.domains:
            d = info["domain"]
            if d.size > 1:
                row = info["done_row"] * d.size
                cu._C.signal_peers_at(info["flag_ptrs"], row, d.rank, step)   # after all my fused kernels (same stream)
                cu._C.wait_flags(info["flags"].data_ptr(), row, d.size, step, d.rank)
        done = torch.cuda.Event()
        done.record(engine.comm_stream)
    torch.cuda.current_stream().wait_event(done)
    for d in engine.domains:
        # a domain of one rank consumed (and cleared) every gradient of its buffer; with peers, each rank read only its
        # shard of every buffer, and clearing a buffer is one local pass in zero_grad() instead of stores over NVLink
        d.grads_clean = d.size == 1 and not st.clip
