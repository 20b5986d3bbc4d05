"""Sharded data-parallel engine: flat parameter / gradient buffers, bucketed gradient
reduction overlapped with backward, optimizer state sharded across the data-parallel
ranks, fused AdamW on fp32 master weights, and the parameter all-gather that feeds
the next forward.

It fills the role of FSDP2 (`fully_shard`) and DDP (`replicate`) in the reference
(reference: train/infra.py:250-346, train/train_qwen.py:195-200, 273-328) with a
layout chosen for 180 GB GPUs on NVSwitch:

* bf16 parameters stay whole on every rank between steps (no per-layer re-gather
  in forward or backward); what is sharded is everything that is 12 of the 16 bytes
  per parameter: fp32 master weights and both Adam moments.
* gradients are reduced ONCE per optimizer step (after the last micro-batch), bucket
  by bucket while backward is still running, by reduce-scatter (``fsdp``) or
  all-reduce (``ddp``).
* the update is one fused kernel per bucket segment on the local shard, writing the
  bf16 parameter shard straight into the flat parameter buffer, followed by an
  all-gather on the communication stream; the next forward waits per bucket, so the
  gather of late buckets overlaps the first layers.
* with ``fused_comm`` the three steps (reduce-scatter, AdamW, all-gather) run as ONE
  kernel over NVLink peer memory (see :mod:`vlm_training_b200.parallel.fused`).

``reshard`` (``training.reshard_params``, the ZeRO-3 form of ``fsdp``): bf16 parameters and gradients are sharded too.
Every rank keeps only its 1/dp shard of each bucket between uses; buckets are cut at the boundaries of "units" (a
decoder layer, a ViT block; everything else forms an always-resident root unit).  A unit's parameter buckets are
all-gathered into buffers that exist only while the unit runs (before its forward, before its recomputation / backward)
and their storage is released afterwards; its gradient buckets exist from the unit's backward until their reduce-scatter
into the gradient shard has been issued.  Autograd keeps references to a bucket's storage object, not to its bytes, so
the storage can be emptied and refilled between forward and backward.

Two reduction domains exist under tensor parallelism: parameters that are split
across TP ranks reduce over the data-parallel group only; parameters replicated
across TP ranks reduce over the whole (dp x tp) world, because with sequence
parallelism every TP rank holds a partial gradient for them.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

ALIGN = 6720  # lcm(1..8) * 8 elements: every shard boundary for dp <= 8 stays 16-byte aligned


@dataclass
class GroupSpec:
    """One optimizer parameter group (learning rate multiplier is applied by the scheduler)."""

    name: str
    params: list
    lr: float
    weight_decay: float = 0.0
    base_lr: float = 0.0

    def __post_init__(self):
        self.base_lr = self.lr


@dataclass
class _Segment:
    start: int
    end: int
    group: int


@dataclass
class _Bucket:
    start: int  # offsets into the domain's flat buffers (elements)
    end: int
    params: list = field(default_factory=list)
    segments: list = field(default_factory=list)
    pending: int = 0
    seen: set = field(default_factory=set)  # ids of the parameters whose gradient has been reported this step
    reduced: bool = False
    gather_event: object = None
    reduce_event: object = None
    unit: int = -1          # reshard mode: index of the unit whose parameters this bucket holds (-1: root, always resident)
    index: int = 0


class _PendingWeightGather:
    """A weight whose part of the unit's parameter gather was left out because the GEMM that consumes it first gathers it
    itself (``gemm_sm100.cu``, weight-gather mode: peer loads of every owner's part into the local bucket, under the tiles
    that run on this rank's own part).  ``run`` is that GEMM; ``finish`` is the plain pull for a consumer that cannot
    take it (another layout, an epilogue)."""

    RUNS = {"gemm": 0, "pull": 0}   # how often a weight arrived inside its GEMM / by the plain pull (tests read it)

    def __init__(self, domain, index, param, lo, ptrs, shard_numel, epoch):
        self.domain, self.index, self.param, self.lo = domain, index, param, lo
        self.ptrs, self.shard_numel, self.epoch = ptrs, shard_numel, epoch

    def run(self, x, w, out, bias):
        from ..ops import cuda as cu

        d = self.domain
        cu._C.gemm_wgather(x, w, out, bias, d.bucket_param[self.index], self.ptrs, self.shard_numel, d.rank, d.f1_sync, self.epoch)
        self.param._vlmt_wgather = None
        self.RUNS["gemm"] += 1

    def finish(self):
        from ..ops import cuda as cu

        d = self.domain
        cu._C.pull_gather_range(self.ptrs, d.bucket_param[self.index], self.shard_numel, self.lo, self.lo + self.param.numel())
        cu._tick()
        self.param._vlmt_wgather = None
        self.RUNS["pull"] += 1


class _Domain:
    """Flat buffers + process group for one reduction domain."""

    def __init__(self, name, entries, group, grad_scale, shard, device, param_dtype, bucket_elems, state_dtype,
                 symmetric=False, reshard=False, unit_of=None):
        self.name, self.group, self.shard, self.device = name, group, shard, device
        self.size = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if (group is not None and dist.is_initialized()) else 0
        self.grad_scale = grad_scale
        unit = math.lcm(ALIGN, 8 * self.size)
        # ---- layout: buckets of whole parameters, each padded to `unit`
        self.buckets: list[_Bucket] = []
        off = 0
        cur = _Bucket(start=0, end=0)
        self.slots = []  # (param, offset, numel, group_idx)
        self.reshard = bool(reshard) and self.shard and self.size > 1
        unit_of = unit_of if (self.reshard and unit_of is not None) else {}
        if self.reshard:   # the root unit first, then the units in order: a bucket never mixes units
            entries = sorted(entries, key=lambda pg: unit_of.get(pg[0], -1))
        for p, gi in entries:
            n = p.numel()
            off = _round_up(off, 8)  # every parameter starts on a 16-byte boundary (bf16)
            u = unit_of.get(p, -1)
            if cur.params and ((off - cur.start) + n > bucket_elems or (self.reshard and u != cur.unit)):
                off = _round_up(off, unit)
                cur.end = off
                self.buckets.append(cur)
                cur = _Bucket(start=off, end=off)
            if not cur.params:
                cur.unit = u
            self.slots.append((p, off, n, gi))
            if cur.segments and cur.segments[-1].group == gi:
                cur.segments[-1].end = off + n
            else:
                cur.segments.append(_Segment(off, off + n, gi))
            cur.params.append(p)
            off += n
        off = _round_up(off, unit)
        cur.end = off
        if cur.params:
            self.buckets.append(cur)
        self.total = off
        for i, b in enumerate(self.buckets):
            b.index = i
        self.param_bucket = {}
        for b in self.buckets:
            for p in b.params:
                self.param_bucket[p] = b
        self.param_dtype = param_dtype
        if self.reshard:
            self._init_resharded(param_dtype, state_dtype, symmetric)
            return
        # ---- buffers
        alloc = _symmetric_empty if symmetric else (lambda n, dt, dev, grp: torch.zeros(n, dtype=dt, device=dev))
        self.flat_param = alloc(self.total, param_dtype, device, group)
        self.flat_grad = alloc(self.total, param_dtype, device, group)
        self.flat_grad.zero_()
        with torch.no_grad():
            for p, o, n, _ in self.slots:
                self.flat_param[o:o + n].copy_(p.detach().reshape(-1))
                p.data = self.flat_param[o:o + n].view(p.shape)
                p.grad = self.flat_grad[o:o + n].view(p.shape)
                # weight-gradient GEMMs may add into this view directly (ops/cuda.py:_wgrad); valid because every
                # such parameter enters exactly one linear per forward pass
                p._vlmt_grad_in_place = True
        # ---- optimizer state on the local shard of every bucket
        self.master, self.exp_avg, self.exp_avg_sq = [], [], []
        for b in self.buckets:
            lo, hi = self.shard_range(b)
            self.master.append(self.flat_param[lo:hi].float().clone())
            self.exp_avg.append(torch.zeros(hi - lo, dtype=state_dtype, device=device))
            self.exp_avg_sq.append(torch.zeros(hi - lo, dtype=state_dtype, device=device))

    # ------------------------------------------------------------------ sharded parameters and gradients (ZeRO-3)
    def _init_resharded(self, param_dtype, state_dtype, symmetric):
        device, group = self.device, self.group
        alloc = _symmetric_empty if symmetric else (lambda n, dt, dev, grp: torch.zeros(n, dtype=dt, device=dev))
        self.flat_param = self.flat_grad = None
        self.symmetric_shards = bool(symmetric)
        self.bucket_param, self.bucket_grad, self.param_shard, self.grad_shard = [], [], [], []
        self.master, self.exp_avg, self.exp_avg_sq = [], [], []
        self.resident, self.grad_live = [], []
        with torch.no_grad():
            for b in self.buckets:
                n = b.end - b.start
                full = torch.zeros(n, dtype=param_dtype, device=device)
                grad = torch.zeros(n, dtype=param_dtype, device=device)
                for p in b.params:
                    o = self._offset_of(p) - b.start
                    full[o:o + p.numel()].copy_(p.detach().reshape(-1))
                    p.data = full[o:o + p.numel()].view(p.shape)
                    p.grad = grad[o:o + p.numel()].view(p.shape)
                    p._vlmt_grad_in_place = True
                lo, hi = self.shard_range(b)
                shard = alloc(hi - lo, param_dtype, device, group)
                shard.copy_(full[lo - b.start:hi - b.start])
                self.param_shard.append(shard)
                self.grad_shard.append(torch.zeros(hi - lo, dtype=param_dtype, device=device))
                self.master.append(shard.float().clone())
                self.exp_avg.append(torch.zeros(hi - lo, dtype=state_dtype, device=device))
                self.exp_avg_sq.append(torch.zeros(hi - lo, dtype=state_dtype, device=device))
                self.bucket_param.append(full)
                self.bucket_grad.append(grad)
                self.resident.append(True)
                self.grad_live.append(True)
        self._nbytes = [(b.end - b.start) * self.bucket_param[0].element_size() for b in self.buckets]
        # bucket index -> (weight, offset inside the bucket) of the weights gathered inside their first GEMM (set by the engine)
        self.f1, self.f1_epoch = {}, 0
        self.f1_sync = torch.zeros(2 * max(self.size, 1), dtype=torch.int32, device=device) if torch.device(device).type == "cuda" else None
        for b in self.buckets:
            if b.unit >= 0:
                self.release_params(b)
                self.release_grads(b)

    def _offset_of(self, p):
        if not hasattr(self, "_slot_offset"):
            self._slot_offset = {q: o for q, o, _, _ in self.slots}
        return self._slot_offset[p]

    def materialize_params(self, b: _Bucket, fuse: bool = False):
        """Make the bucket's parameters usable: give its storage its bytes back and all-gather the shards into it.
        ``fuse``: leave the bucket's first-consumed weight to the GEMM that reads it (forward passes only)."""
        i = b.index
        if self.resident[i]:
            return
        full = self.bucket_param[i]
        full.untyped_storage().resize_(self._nbytes[i])
        self.resident[i] = True
        self.gather_params(b, fuse)

    def gather_params(self, b: _Bucket, fuse: bool = False):
        i = b.index
        full, shard = self.bucket_param[i], self.param_shard[i]
        ent = self.f1.get(i) if (fuse and self.symmetric_shards and full.is_cuda) else None
        if ent is not None:
            from . import symm
            from ..ops import cuda as cu

            p, lo = ent
            ptrs, n = symm.peer_ptrs(shard), shard.numel()
            cu._C.pull_gather_range(ptrs, full, n, 0, lo)
            cu._C.pull_gather_range(ptrs, full, n, lo + p.numel(), full.numel())
            cu._tick(2)
            self.f1_epoch += 1
            p._vlmt_wgather = _PendingWeightGather(self, i, p, lo, ptrs, n, self.f1_epoch)
            return
        if self.symmetric_shards and full.is_cuda:
            from . import symm
            from ..ops import cuda as cu

            if not hasattr(self, "_no_flags"):
                self._no_flags = torch.zeros(64, dtype=torch.int32, device=self.device)
            # peers' shards are stable between optimizer steps (the engine ends a step with a barrier on the device): a
            # plain peer pull with nothing to wait for (collective number 0 is always "there")
            cu._C.pull_gather(symm.peer_ptrs(shard), full, shard.numel(), self._no_flags.data_ptr(), 0)
            cu._tick()
        else:
            dist.all_gather_into_tensor(full, shard if full.is_cuda else shard.clone(), group=self.group)

    def release_params(self, b: _Bucket):
        i = b.index
        if not self.resident[i] or b.unit < 0:
            return
        t = self.bucket_param[i]
        if t.is_cuda:
            t.record_stream(torch.cuda.current_stream())
        t.untyped_storage().resize_(0)
        self.resident[i] = False

    def materialize_grads(self, b: _Bucket):
        i = b.index
        if self.grad_live[i]:
            return
        g = self.bucket_grad[i]
        g.untyped_storage().resize_(self._nbytes[i])
        g.zero_()
        self.grad_live[i] = True

    def release_grads(self, b: _Bucket, stream=None):
        i = b.index
        if not self.grad_live[i] or b.unit < 0:
            return
        g = self.bucket_grad[i]
        if g.is_cuda and stream is not None:
            g.record_stream(stream)   # the reduce-scatter on that stream may still be reading
        g.untyped_storage().resize_(0)
        self.grad_live[i] = False

    # ------------------------------------------------------------------ layout-independent accessors
    def bucket_grad_view(self, b: _Bucket):
        return self.bucket_grad[b.index] if self.reshard else self.flat_grad[b.start:b.end]

    def shard_grad_view(self, b: _Bucket, s: int, e: int):
        """Elements [s, e) (domain offsets, inside this rank's shard of ``b``) of the reduced gradient."""
        if self.reshard:
            lo, _ = self.shard_range(b)
            return self.grad_shard[b.index][s - lo:e - lo]
        return self.flat_grad[s:e]

    def shard_param_view(self, b: _Bucket, s: int, e: int):
        if self.reshard:
            lo, _ = self.shard_range(b)
            return self.param_shard[b.index][s - lo:e - lo]
        return self.flat_param[s:e]

    def shard_range(self, b: _Bucket):
        if not self.shard or self.size == 1:
            return b.start, b.end
        n = (b.end - b.start) // self.size
        return b.start + self.rank * n, b.start + (self.rank + 1) * n


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _symmetric_empty(n, dtype, device, group):
    from .symm import symmetric_zeros

    return symmetric_zeros(n, dtype, device, group)


def _find_units(model, group_of):
    """Units of parameter residency: every element of an ``nn.ModuleList`` that holds trainable parameters (decoder
    layers, ViT blocks, DeepStack mergers).  Returns ``(modules, {parameter: unit index})``; parameters outside any
    unit belong to the root unit (-1), which stays resident."""
    import torch.nn as nn

    units, unit_of = [], {}
    for mod in model.modules():
        if isinstance(mod, nn.ModuleList):
            for child in mod:
                ps = [p for p in child.parameters() if p in group_of and p not in unit_of]
                if not ps:
                    continue
                for p in ps:
                    unit_of[p] = len(units)
                units.append(child)
    return units, unit_of


class ShardedOptimizerEngine(torch.optim.Optimizer):
    """Owns the model's trainable parameters as flat buffers and performs
    gradient synchronisation + AdamW + parameter redistribution.

    ``step()`` = finish gradient reduction → (optional clip) → fused AdamW on shards →
    all-gather parameters.  ``zero_grad()`` clears the flat gradient buffers.
    ``param_groups`` mimics ``torch.optim.Optimizer.param_groups`` enough for
    ``LambdaLR`` (keys ``lr`` / ``initial_lr``)."""

    def __init__(self, model, groups: list[GroupSpec], *, dp_group=None, world_group=None, tp_size: int = 1,
                 mode: str = "fsdp", betas=(0.9, 0.999), eps: float = 1e-8, max_grad_norm: float | None = None,
                 bucket_mb: float = 256.0, state_dtype=torch.float32, fused_comm: bool = False, overlap: bool = True,
                 reshard: bool = False, reshard_after_forward: bool = True, fuse_first_gemm: bool = True):
        pgs = [{"params": list(g.params), "lr": g.lr, "weight_decay": g.weight_decay, "name": g.name} for g in groups]
        super().__init__(pgs, defaults={"lr": groups[0].lr, "weight_decay": 0.0})
        self.model = model
        self.groups = groups
        self.betas, self.eps, self.max_grad_norm = betas, eps, max_grad_norm
        self.mode = mode
        self.step_count = 0
        self.fused_comm = fused_comm
        self.overlap = overlap
        params = [p for g in groups for p in g.params]
        if not params:
            raise ValueError("no trainable parameters")
        device = params[0].device
        self.device = device
        self.is_cuda = device.type == "cuda"
        pdtype = params[0].dtype
        group_of = {p: gi for gi, g in enumerate(groups) for p in g.params}
        dp_size = dist.get_world_size(dp_group) if (dist.is_initialized() and dp_group is not None) else (
            dist.get_world_size() if dist.is_initialized() and tp_size == 1 else 1)
        self.dp_size = dp_size
        shard = mode == "fsdp"
        bucket_elems = int(bucket_mb * (1 << 20) / params[0].element_size())
        # parameter order = registration order (≈ forward order): late buckets finish first in backward
        ordered = [p for p in model.parameters() if p in group_of]
        experts = [(p, group_of[p]) for p in ordered if getattr(p, "_ep_sharded", False)]
        ordered = [p for p in ordered if not getattr(p, "_ep_sharded", False)]
        sharded = [(p, group_of[p]) for p in ordered if getattr(p, "_tp_sharded", False)]
        replicated = [(p, group_of[p]) for p in ordered if not getattr(p, "_tp_sharded", False)]
        self.domains: list[_Domain] = []
        self.comm_path = "local" if not dist.is_initialized() else "nccl"
        reason = ""
        self.reshard = bool(reshard) and shard and dist.is_initialized() and dp_size > 1
        self.reshard_after_forward = reshard_after_forward
        self.units, unit_of = [], {}
        symmetric_shards = False
        if self.reshard:
            self.units, unit_of = _find_units(model, group_of)
            # with `fused_comm` the parameter shards live in symmetric memory and a unit's parameters are gathered by
            # our own peer-pull kernel; the gradient side is a reduce-scatter into the shard in both cases
            symmetric_shards = bool(fused_comm) and self.is_cuda
            if fused_comm:
                fused_comm, reason = False, "sharded parameters and gradients use reduce-scatter into shards, not the one-kernel step"
        if fused_comm and self.is_cuda and dist.is_initialized():
            # decided before the buffers are allocated: the one-kernel path needs them in symmetric memory
            if state_dtype not in (torch.float32, torch.bfloat16):
                fused_comm, reason = False, f"the fused kernel keeps fp32 or bf16 Adam moments, optimizer_state_dtype is {state_dtype}"
        symmetric = fused_comm and self.is_cuda and dist.is_initialized()
        if experts:
            # expert-parallel parameters: each rank owns different experts, whose gradients already hold the
            # contributions of every rank of the all-to-all group; they are summed only over the ranks that own
            # the same experts (none when ep_size equals the data-parallel size)
            ep = getattr(model, "_ep_ctx", None)
            rep_group = ep.replica_group if (ep is not None and ep.replica_size > 1) else None
            self.domains.append(_Domain("ep_experts", experts, rep_group, 1.0 / dp_size, shard and rep_group is not None, device,
                                        pdtype, bucket_elems, state_dtype, symmetric and rep_group is not None))
        if tp_size > 1:
            if sharded:
                self.domains.append(_Domain("tp_sharded", sharded, dp_group, 1.0 / dp_size, shard, device, pdtype,
                                            bucket_elems, state_dtype, symmetric or symmetric_shards, self.reshard, unit_of))
            if replicated:
                with torch.no_grad():
                    self._identical = [p for p, _ in replicated if getattr(p, "_tp_grad", "partial") == "identical"]
                self.domains.append(_Domain("tp_replicated", replicated, world_group, 1.0 / dp_size, shard, device, pdtype,
                                            bucket_elems, state_dtype, symmetric or symmetric_shards, self.reshard, unit_of))
            self._identical_scale = 1.0 / tp_size
        else:
            self._identical = []
            self.domains.append(_Domain("all", replicated + sharded, dp_group if dp_group is not None else world_group,
                                        1.0 / dp_size, shard, device, pdtype, bucket_elems, state_dtype,
                                        symmetric or symmetric_shards, self.reshard, unit_of))
        self.comm_stream = torch.cuda.Stream(device=device) if self.is_cuda else None
        self.gather_stream = torch.cuda.Stream(device=device) if self.is_cuda else None
        self._hooks = []
        self._sync_grads = True
        self._fused = None
        if symmetric:
            from . import fused

            ok, reason = fused.usable(self)
            if ok:
                self._fused = fused.FusedStepState(self)
                self.comm_path = "fused"
        if self.reshard:
            import logging

            logging.getLogger("vlm_training_b200").info(
                f"parameters and gradients are sharded over {dp_size} data-parallel ranks: {len(self.units)} units, "
                f"{sum(len(d.buckets) for d in self.domains if d.reshard)} buckets, "
                f"{'own peer-pull' if symmetric_shards else 'library all-gather'} for the parameter gathers")
        if dist.is_initialized() and self.is_cuda:
            import logging

            logging.getLogger("vlm_training_b200").info(
                "optimizer step: " + ("reduce-scatter + AdamW + all-gather in one NVLink kernel per bucket" if self._fused is not None
                                      else f"NCCL reduce-scatter / all-gather around the AdamW kernel ({reason or 'fused_comm is off'})"))
        # one process on a GPU, no clipping: a bucket's AdamW runs on the side stream as soon as backward has finished the bucket
        # AFTER it (one bucket of lag: every kernel that reads the bucket's weights has been enqueued by then), so the
        # memory-bound update hides under the compute-bound rest of backward instead of running after it
        tied = bool(getattr(getattr(getattr(model, "config", None), "text", None), "tie_word_embeddings", False))
        self._early = (self.is_cuda and overlap and not dist.is_initialized() and max_grad_norm is None and not self.reshard
                       and not tied and pdtype == torch.bfloat16 and os.environ.get("VLMT_EARLY_ADAMW", "1") != "0")
        self._early_prev = None     # (domain, bucket) complete but not yet updated
        if (self.is_cuda and overlap and dist.is_initialized()) or self.reshard or self._early:
            self._install_hooks()
        self._bwd_phase, self._prefetched = False, -1
        self.fuse_first_gemm = False
        if self.reshard:
            if fuse_first_gemm and symmetric_shards and tp_size == 1:
                self._pick_fused_weights()
            self._install_unit_hooks()
        if self.is_cuda:
            self._install_forward_waits()
        self._clip_buf = torch.zeros(1, dtype=torch.float32, device=device)
        self._barrier_buf = torch.zeros(1, dtype=torch.float32, device=device)
        self.last_grad_norm = None

    # ------------------------------------------------------------------ torch.optim surface
    def zero_grad(self, set_to_none: bool = False):
        for d in self.domains:
            if d.reshard:
                clean = getattr(d, "grads_clean", False)
                d.grads_clean = False
                for b in d.buckets:
                    if not clean:
                        d.grad_shard[b.index].zero_()
                    if b.unit < 0:
                        d.bucket_grad[b.index].zero_()
            elif getattr(d, "grads_clean", False):
                d.grads_clean = False  # the AdamW kernel of the last step() cleared every gradient it consumed
            elif self.is_cuda:
                from ..ops import cuda as cu

                cu.memset_zero_(d.flat_grad)
            else:
                d.flat_grad.zero_()
            for b in d.buckets:
                b.pending = len(b.params)
                b.seen.clear()
                b.reduced = False
                b.reduce_event = None

    def set_requires_gradient_sync(self, flag: bool):
        """False on all but the last micro-batch of an accumulation window."""
        self._sync_grads = flag

    # ------------------------------------------------------------------ overlap plumbing
    def _install_hooks(self):
        for d in self.domains:
            for b in d.buckets:
                b.pending = len(b.params)
                for p in b.params:
                    hook = self._make_hook(d, b)
                    p._vlmt_grad_ready = hook
                    self._hooks.append(p.register_post_accumulate_grad_hook(hook))

    def _make_hook(self, d, b):
        def hook(p):
            if not self._sync_grads and not d.reshard:
                return
            # once per parameter and step: a weight-gradient GEMM that adds into the flat buffer itself reports the
            # parameter by hand (`_vlmt_grad_ready`), and autograd may report it again with nothing to accumulate
            if id(p) in b.seen:
                return
            b.seen.add(id(p))
            b.pending -= 1
            if b.pending == 0 and not b.reduced and self._early:
                b.reduced = True
                prev, self._early_prev = self._early_prev, (d, b)
                if prev is not None:
                    self._early_update(*prev)
                return
            if b.pending == 0 and not b.reduced:
                if self._fused is not None:
                    from . import fused

                    fused.process_bucket(self, d, d.buckets.index(b))
                else:
                    self._reduce_bucket(d, b)
        return hook

    def _install_forward_waits(self):
        """Before a module's forward, wait for the all-gather of the buckets that hold its parameters."""
        engine = self

        def pre_hook(mod, _args):
            for p in mod._parameters.values():
                if p is None:
                    continue
                for d in engine.domains:
                    b = d.param_bucket.get(p)
                    if b is not None and b.gather_event is not None:
                        torch.cuda.current_stream().wait_event(b.gather_event)
                        b.gather_event = None
        for mod in self.model.modules():
            if any(p is not None for p in mod._parameters.values()):
                self._hooks.append(mod.register_forward_pre_hook(pre_hook))

    # ------------------------------------------------------------------ residency of sharded parameters (reshard mode)
    def _unit_buckets(self, u: int):
        for d in self.domains:
            if d.reshard:
                for b in d.buckets:
                    if b.unit == u:
                        yield d, b

    def _enter_unit(self, u: int, backward: bool):
        """Unit ``u`` is about to run: its parameters become resident (and, before a backward pass, its gradient buckets);
        the other units' parameters are released unless forward passes keep them (``reshard_after_forward`` off); the
        unit that runs next (the following one in a forward pass, the preceding one in a backward pass) is gathered on
        the communication stream meanwhile."""
        if backward:
            self._bwd_phase = True
        if backward or self.reshard_after_forward:
            for d in self.domains:
                if d.reshard:
                    for b in d.buckets:
                        if b.unit >= 0 and b.unit != u and not (b.gather_event is not None and b.unit == self._prefetched):
                            d.release_params(b)
        for d, b in self._unit_buckets(u):
            if b.gather_event is not None:   # gathered ahead of time on the communication stream
                if self.is_cuda:
                    torch.cuda.current_stream().wait_event(b.gather_event)
                    d.bucket_param[b.index].record_stream(torch.cuda.current_stream())
                b.gather_event = None
            d.materialize_params(b, fuse=self.fuse_first_gemm and not self._bwd_phase)
            if backward:
                d.materialize_grads(b)
        nxt = u - 1 if self._bwd_phase else u + 1
        if self.is_cuda and 0 <= nxt < len(self.units) and (backward or not self._bwd_phase):
            self._prefetched = nxt
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            with torch.cuda.stream(self.gather_stream):   # its own stream: never queued behind a gradient reduce-scatter
                self.gather_stream.wait_event(ev)
                for d, b in self._unit_buckets(nxt):
                    if not d.resident[b.index]:
                        d.materialize_params(b, fuse=self.fuse_first_gemm and not self._bwd_phase)
                        b.gather_event = torch.cuda.Event()
                        b.gather_event.record(self.gather_stream)

    # weights gathered by the GEMM that consumes them first (the fused projections at the top of a block)
    FIRST_GEMM_SUFFIXES = ("qkv.weight", "in_proj.weight")

    def _pick_fused_weights(self):
        """Per unit, the weight of its first GEMM: its part of the unit's parameter gather moves into that GEMM."""
        names = {p: n for n, p in self.model.named_parameters()}
        picked = 0
        for d in self.domains:
            if not d.reshard or d.f1_sync is None:
                continue
            units_done = set()
            for b in d.buckets:
                if b.unit < 0 or b.unit in units_done:
                    continue
                for p in b.params:
                    n = names.get(p, "")
                    if (n.endswith(self.FIRST_GEMM_SUFFIXES) and p.dim() == 2 and p.dtype == torch.bfloat16 and p.shape[0] > 128
                            and p.shape[1] % 8 == 0 and p.numel() % 8 == 0 and not getattr(p, "_vlmt_fp8", False)):
                        d.f1[b.index] = (p, d._offset_of(p) - b.start)
                        units_done.add(b.unit)
                        picked += 1
                        break
        self.fuse_first_gemm = picked > 0
        if picked:
            import logging

            logging.getLogger("vlm_training_b200").info(f"{picked} units gather the weight of their first GEMM inside that GEMM")

    def _check_consumed(self, u: int):
        for d, b in self._unit_buckets(u):
            ent = d.f1.get(b.index)
            if ent is not None and getattr(ent[0], "_vlmt_wgather", None) is not None:
                raise RuntimeError("a weight that was left to its first GEMM to gather was not read by a GEMM in this forward pass; "
                                   "switch training.reshard_fuse_first_gemm off for this model")

    def _install_unit_hooks(self):
        for u, mod in enumerate(self.units):
            if self.fuse_first_gemm:
                self._hooks.append(mod.register_forward_hook(lambda m, a, o, u=u: self._check_consumed(u)))
            self._hooks.append(mod.register_forward_pre_hook(lambda m, a, u=u: self._enter_unit(u, False)))
            self._hooks.append(mod.register_full_backward_pre_hook(lambda m, g, u=u: self._enter_unit(u, True)))

    def release_all(self):
        for d in self.domains:
            if d.reshard:
                for b in d.buckets:
                    if b.gather_event is not None and self.is_cuda:
                        torch.cuda.current_stream().wait_event(b.gather_event)
                    b.gather_event = None
                    d.release_params(b)

    def all_resident(self):
        """Context manager: every parameter is whole while it is active (checkpoints, evaluation, weight surgery)."""
        engine = self

        class _Ctx:
            def __enter__(self_inner):
                for d in engine.domains:
                    if d.reshard:
                        for b in d.buckets:
                            d.materialize_params(b)
                return engine

            def __exit__(self_inner, *exc):
                engine.release_all()
                return False
        return _Ctx()

    def wait_all_gathers(self):
        if not self.is_cuda:
            return
        for d in self.domains:
            for b in d.buckets:
                if b.gather_event is not None:
                    torch.cuda.current_stream().wait_event(b.gather_event)
                    b.gather_event = None

    # ------------------------------------------------------------------ gradient reduction
    def _reduce_bucket(self, d: _Domain, b: _Bucket):
        b.reduced = True
        if d.size == 1 or not dist.is_initialized():
            return
        if d.reshard:
            d.materialize_grads(b)   # a bucket none of whose parameters got a gradient this pass: zeros
        g = d.bucket_grad_view(b)
        if self._identical and d.name == "tp_replicated":
            for p in b.params:
                if getattr(p, "_tp_grad", "partial") == "identical":
                    p.grad.mul_(self._identical_scale)
        if self.is_cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                self._collective_reduce(d, b, g)
                b.reduce_event = torch.cuda.Event()
                b.reduce_event.record(self.comm_stream)
            if d.reshard:
                d.release_grads(b, stream=self.comm_stream)
        else:
            self._collective_reduce(d, b, g)
            if d.reshard:
                d.release_grads(b)
        if d.reshard:   # ready for the next micro-batch of the accumulation window
            b.pending = len(b.params)
            b.seen.clear()
            b.reduced = False

    def _collective_reduce(self, d, b, g):
        if d.reshard:
            # reduce-scatter into a temporary, added to the gradient shard (micro-batches of an accumulation window
            # are reduced one by one: the full-size gradients do not outlive their unit's backward pass)
            lo, hi = d.shard_range(b)
            shard = d.grad_shard[b.index]
            if g.is_cuda:
                tmp = torch.empty_like(shard)
                dist.reduce_scatter_tensor(tmp, g, op=dist.ReduceOp.SUM, group=d.group)
                shard.add_(tmp)
            else:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=d.group)
                shard.add_(g[lo - b.start:hi - b.start])
            if b.unit < 0:
                g.zero_()   # the root unit's gradient buckets stay allocated: ready for the next pass
            return
        if d.shard and g.is_cuda:
            lo, hi = d.shard_range(b)
            dist.reduce_scatter_tensor(d.flat_grad[lo:hi], g, op=dist.ReduceOp.SUM, group=d.group)
        else:
            # ddp mode, and gloo (which has no reduce-scatter): all-reduce the bucket
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=d.group)

    def finish_grad_sync(self):
        for d in self.domains:
            for b in d.buckets:
                if d.reshard and not b.seen:
                    continue   # nothing left to reduce: complete buckets were reduced (and reset) by the gradient hooks
                if not b.reduced:
                    self._reduce_bucket(d, b)
        if self.is_cuda:
            for d in self.domains:
                for b in d.buckets:
                    if b.reduce_event is not None:
                        torch.cuda.current_stream().wait_event(b.reduce_event)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        if self._fused is not None:
            from . import fused

            fused.finish_step(self)  # buckets not reached by the hooks + the all-ranks-done round
            self.step_count += 1
            return
        self.step_count += 1
        self.finish_grad_sync()
        clip = 1.0
        if self.max_grad_norm is not None:
            clip = self._clip_coefficient()
        b1, b2 = self.betas
        if self._early:
            self._early_prev = None   # the last complete bucket and the buckets backward never completed: updated below
        for d in self.domains:
            for bi, b in enumerate(d.buckets):
                if getattr(b, "early_done", False):
                    b.early_done = False
                    continue
                lo, hi = d.shard_range(b)
                for seg in b.segments:
                    s, e = max(seg.start, lo), min(seg.end, hi)
                    if e <= s:
                        continue
                    pg = self.param_groups[seg.group]
                    self._adamw(d, bi, s - lo, e - lo, d.shard_grad_view(b, s, e), d.shard_param_view(b, s, e), pg["lr"],
                                pg["weight_decay"], b1, b2, d.grad_scale * clip)
                if not d.reshard:
                    self._gather_bucket(d, b)
            if d.reshard:
                # every rank's shards are final before anybody gathers from them again (one tiny stream-ordered collective),
                # then the always-resident root unit gets its new parameters
                if dist.is_initialized() and d.size > 1:
                    dist.all_reduce(self._barrier_buf, group=d.group)
                for b in d.buckets:
                    if b.unit < 0:
                        d.gather_params(b)
                d.grads_clean = self.is_cuda and d.param_dtype == torch.bfloat16
                continue
            # on this path every rank's kernel clears the gradients it consumed; when each rank consumes the whole
            # buffer (one rank, or unsharded data parallelism) the next zero_grad() has nothing left to do
            d.grads_clean = self.is_cuda and d.flat_param.dtype == torch.bfloat16 and (d.size == 1 or not d.shard)
        if self.reshard:
            self.release_all()
            self._bwd_phase, self._prefetched = False, -1
        if self._early:
            torch.cuda.current_stream().wait_stream(self.comm_stream)   # the updates that ran under backward

    def _early_update(self, d, b):
        """AdamW of a bucket whose gradients are final, on the side stream, ordered after everything enqueued so far."""
        b1, b2 = self.betas
        bi = b.index
        lo, hi = d.shard_range(b)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            for seg in b.segments:
                s, e = max(seg.start, lo), min(seg.end, hi)
                if e <= s:
                    continue
                pg = self.param_groups[seg.group]
                self._adamw(d, bi, s - lo, e - lo, d.shard_grad_view(b, s, e), d.shard_param_view(b, s, e), pg["lr"],
                            pg["weight_decay"], b1, b2, d.grad_scale, step=self.step_count + 1)
        b.early_done = True

    def _adamw(self, d, bi, s, e, grad, param, lr, wd, b1, b2, grad_scale, step=None):
        master, m, v = d.master[bi][s:e], d.exp_avg[bi][s:e], d.exp_avg_sq[bi][s:e]
        step = self.step_count if step is None else step
        if self.is_cuda and param.dtype == torch.bfloat16:
            from ..ops import cuda as cu

            cu.adamw_step_(grad, master, m, v, param, lr, b1, b2, self.eps, wd, step, grad_scale, zero_grad=True)
            return
        g = grad.float() * grad_scale
        mf, vf = m.float(), v.float()
        mf.mul_(b1).add_(g, alpha=1 - b1)
        vf.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        master.mul_(1 - lr * wd)
        master.addcdiv_(mf / bc1, (vf / bc2).sqrt_().add_(self.eps), value=-lr)
        m.copy_(mf)
        v.copy_(vf)
        param.copy_(master)

    def _gather_bucket(self, d: _Domain, b: _Bucket):
        if not d.shard or d.size == 1 or not dist.is_initialized():
            return
        lo, hi = d.shard_range(b)
        if self.is_cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                dist.all_gather_into_tensor(d.flat_param[b.start:b.end], d.flat_param[lo:hi], group=d.group)
                b.gather_event = torch.cuda.Event()
                b.gather_event.record(self.comm_stream)
        else:
            shard = d.flat_param[lo:hi].clone()
            dist.all_gather_into_tensor(d.flat_param[b.start:b.end], shard, group=d.group)

    def _clip_coefficient(self) -> float:
        """Global gradient norm over every reduced shard (each element counted once) → clip factor."""
        self._clip_buf.zero_()
        for d in self.domains:
            for b in d.buckets:
                lo, hi = d.shard_range(b)
                g = d.shard_grad_view(b, lo, hi)
                if self.is_cuda and g.dtype in (torch.bfloat16, torch.float32):
                    from ..ops import cuda as cu

                    part = torch.zeros(1, dtype=torch.float32, device=self.device)
                    cu.sumsq_(g, part)
                else:
                    part = g.float().pow(2).sum().reshape(1)
                self._clip_buf += part * (d.grad_scale ** 2) / (1 if d.shard else d.size)
        if dist.is_initialized():
            dist.all_reduce(self._clip_buf)
            if self.domains[0].name == "tp_sharded":
                pass  # shards are disjoint across the world in both domains: a plain sum is exact
        norm = float(self._clip_buf.sqrt().item())
        self.last_grad_norm = norm
        return min(1.0, self.max_grad_norm / (norm + 1e-6))

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        out = {"step": self.step_count, "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}
        for d in self.domains:
            out[d.name] = {
                "master": torch.cat(d.master), "exp_avg": torch.cat(d.exp_avg), "exp_avg_sq": torch.cat(d.exp_avg_sq),
                "layout": {"total": d.total, "size": d.size, "rank": d.rank, "shard": d.shard,
                           "buckets": [(b.start, b.end) for b in d.buckets]}}
        return out

    def load_state_dict(self, state: dict):
        self.step_count = int(state["step"])
        for pg, saved in zip(self.param_groups, state["param_groups"]):
            pg.update({k: v for k, v in saved.items() if k in ("lr", "initial_lr", "weight_decay")})
        for d in self.domains:
            s = state[d.name]
            for name, dst in (("master", d.master), ("exp_avg", d.exp_avg), ("exp_avg_sq", d.exp_avg_sq)):
                off = 0
                for t in dst:
                    t.copy_(s[name][off:off + t.numel()])
                    off += t.numel()
        self.params_from_master()

    def params_from_master(self):
        """The bf16 parameters follow the fp32 master copy (after loading optimizer state)."""
        with torch.no_grad():
            for d in self.domains:
                for bi, b in enumerate(d.buckets):
                    lo, hi = d.shard_range(b)
                    d.shard_param_view(b, lo, hi).copy_(d.master[bi])
                    if d.reshard:
                        if d.resident[b.index]:
                            d.gather_params(b)
                    else:
                        self._gather_bucket(d, b)
        self.wait_all_gathers()

    def resync_master_from_params(self):
        """Re-read the master weights from the (bf16) parameters, e.g. after loading a model checkpoint (in reshard mode
        inside ``all_resident()``: the parameters must be whole to be read)."""
        with torch.no_grad():
            for d in self.domains:
                for bi, b in enumerate(d.buckets):
                    lo, hi = d.shard_range(b)
                    if d.reshard:
                        d.param_shard[b.index].copy_(d.bucket_param[b.index][lo - b.start:hi - b.start])
                    d.master[bi].copy_(d.shard_param_view(b, lo, hi))

    def memory_bytes(self) -> dict:
        tot = {"param": 0, "grad": 0, "optimizer": 0}
        for d in self.domains:
            if d.reshard:   # what is held right now: shards plus the buckets whose storage is live
                for i in range(len(d.buckets)):
                    tot["param"] += d.param_shard[i].numel() * d.param_shard[i].element_size() + d.bucket_param[i].untyped_storage().size()
                    tot["grad"] += d.grad_shard[i].numel() * d.grad_shard[i].element_size() + d.bucket_grad[i].untyped_storage().size()
                continue
            tot["param"] += d.flat_param.numel() * d.flat_param.element_size()
            tot["grad"] += d.flat_grad.numel() * d.flat_grad.element_size()
            for t in d.master + d.exp_avg + d.exp_avg_sq:
                tot["optimizer"] += t.numel() * t.element_size()
        return tot
