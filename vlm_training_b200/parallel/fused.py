"""One-kernel NVLink paths used by the sharded optimizer engine and tensor parallelism.

``fused_reduce_adamw_gather`` replaces, per bucket, the sequence
``reduce_scatter(grads) → AdamW(shard) → all_gather(params)`` (three passes over HBM and
two NCCL kernels) by a single kernel that pulls the gradient shard from every peer (or one
in-switch ``multimem.ld_reduce``), updates the fp32 state and pushes the bf16 parameters to
every peer (``vlm_training_b200/ops/csrc/comm_kernels.cu``).  It needs the engine's flat
buffers to live in symmetric memory (``fused_comm=True``).

Ordering: a rank may start a bucket only after EVERY rank has finished writing that bucket's
gradients, and nobody may read parameters until every rank's pushes have landed.  Both
conditions are established with a one-element NCCL all-reduce on the communication stream —
no spin-waits in our own kernels.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import symm


def fused_reduce_adamw_gather(engine) -> bool:
    """Run the optimizer step through the fused kernel.  Returns False when the engine's buffers
    are not symmetric (the caller then takes the NCCL path)."""
    from ..ops import cuda as cu

    domains = [d for d in engine.domains]
    if any(d.size > 1 and symm.handle_of(d.flat_grad) is None for d in domains):
        return False
    b1, b2 = engine.betas
    step = engine.step_count
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    cur = torch.cuda.current_stream()
    comm = engine.comm_stream
    token = engine.__dict__.setdefault("_sync_token", torch.zeros(1, device=engine.device))
    # every rank's backward (all gradient writes) must be complete before anyone pulls
    ev = torch.cuda.Event()
    ev.record(cur)
    with torch.cuda.stream(comm):
        comm.wait_event(ev)
        for d in domains:
            if d.size > 1:
                dist.all_reduce(token, group=d.group)
        for d in domains:
            world = d.size
            if world > 1:
                g_ptrs, p_ptrs = symm.peer_ptrs(d.flat_grad), symm.peer_ptrs(d.flat_param)
                g_mc, p_mc = symm.multicast_ptr(d.flat_grad), symm.multicast_ptr(d.flat_param)
            else:
                g_ptrs, p_ptrs, g_mc, p_mc = [d.flat_grad.data_ptr()], [d.flat_param.data_ptr()], 0, 0
            esz = d.flat_grad.element_size()
            for bi, b in enumerate(d.buckets):
                if engine._identical and d.name == "tp_replicated":
                    for p in b.params:
                        if getattr(p, "_tp_grad", "partial") == "identical":
                            p.grad.mul_(engine._identical_scale)
                lo, hi = d.shard_range(b)
                for seg in b.segments:
                    s, e = max(seg.start, lo), min(seg.end, hi)
                    if e <= s:
                        continue
                    # parameters start on 8-element boundaries; a segment's tail may not end on one: the padding
                    # behind it holds zero gradients, so rounding the end up is harmless
                    e = min(hi, (e + 7) // 8 * 8)
                    pg = engine.param_groups[seg.group]
                    cu._C.fused_rs_adamw_ag(
                        [p + b.start * esz for p in g_ptrs], [p + b.start * esz for p in p_ptrs],
                        (g_mc + b.start * esz) if g_mc else 0, (p_mc + b.start * esz) if p_mc else 0,
                        world, s - b.start, e - b.start, d.master[bi], d.exp_avg[bi], d.exp_avg_sq[bi], s - lo,
                        pg["lr"], b1, b2, engine.eps, pg["weight_decay"], bc1, bc2, d.grad_scale)
                    cu._tick()
                b.reduced = True
        for d in domains:
            if d.size > 1:
                dist.all_reduce(token, group=d.group)  # all pushes have landed everywhere
        done = torch.cuda.Event()
        done.record(comm)
    cur.wait_event(done)
    return True
