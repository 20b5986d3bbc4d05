"""Expert parallelism for the sparse MoE block: every rank of the expert-parallel group owns ``E / ep``
consecutive experts; routed tokens travel to the owner of their expert (all-to-all dispatch), run through the
local experts as one grouped computation, and travel back (all-to-all combine), where the routing weights are
applied in a fixed slot order so the result does not depend on arrival order.

The reference has no expert parallelism (its MoE model runs every expert on every rank, reference:
models/qwen3_5/model.py:715-751); this is an addition for the 256-expert configuration.

Two transports.  ``dist``: ``all_to_all_single`` on the process group (gloo on CPU, NCCL on GPUs) with one host read
per layer for the split sizes.  ``fused`` (GPUs, symmetric memory, :class:`EPFused`): no host read and no library
collective — every rank pushes its per-expert counts to its peers, computes from the complete count matrix the row
that each of its slots gets inside the OWNER's padded expert buffer, and stores the token rows straight into the
owner's memory over NVLink (``csrc/moe_kernels.cu``); the owner runs the grouped tcgen05 GEMMs on what arrived and
stores every output row back into the source rank's per-slot buffer, where the weighted sum runs in slot order.
Ordering is by flags with bounded waits, as for the tensor-parallel collectives.

The expert-parallel group is the data-parallel group (``ep_size == dp``) or a contiguous sub-group of it
(``ep_size`` divides ``dp``): ranks in one group see different data.  Expert parameters are tagged
``_ep_sharded`` so that the optimizer engine reduces their gradients only over the ranks that hold the same experts.
``state_dict()`` still shows full ``[E, ...]`` expert tensors (all-gather on save, slice on load) so checkpoints and
HF snapshots do not depend on the expert-parallel size.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class EPContext:
    group: object = None     # ranks that share one set of tokens' experts (all-to-all partners)
    size: int = 1
    rank: int = 0
    replica_group: object = None  # ranks that own the same experts (gradient reduction for expert parameters)
    replica_size: int = 1
    n_experts: int = 0
    fused: object = None     # EPFused when tokens travel by peer stores

    @property
    def local_experts(self) -> int:
        return self.n_experts // self.size


class _AllToAllRows(torch.autograd.Function):
    """Variable-size all-to-all on rows; the backward is the all-to-all with the split lists exchanged."""

    @staticmethod
    def forward(fctx, x, in_splits, out_splits, group):
        fctx.in_splits, fctx.out_splits, fctx.group = in_splits, out_splits, group
        x = x.contiguous()
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(fctx, g):
        g = g.contiguous()
        out = g.new_empty((sum(fctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g, output_split_sizes=fctx.in_splits, input_split_sizes=fctx.out_splits, group=fctx.group)
        return out, None, None, None


class EPFused:
    """Peer-memory state of one expert-parallel group: flags, the count matrix, the buffer that receives dispatched rows
    (forward: token rows, backward: output-gradient rows), the per-slot buffer that receives returned rows, and the
    number of the current exchange.  Buffers are sized on first use; a row capacity of ``VLMT_EP_CAPACITY`` (default 2)
    times the mean load bounds what a rank can receive — an owner that would exceed it sets status 200."""

    def __init__(self, ep: EPContext, device):
        import os

        from . import symm

        self.ep, self.device = ep, device
        self.capacity = float(os.environ.get("VLMT_EP_CAPACITY", "2.0"))
        self.flags = symm.symmetric_zeros(64, torch.int32, device, ep.group)
        self.flag_ptrs = symm.peer_ptrs(self.flags)
        self.counts = symm.symmetric_zeros(ep.size * ep.n_experts, torch.int32, device, ep.group)
        self.counts_ptrs = symm.peer_ptrs(self.counts)
        symm.apply_flag_wait_limit()
        self.epoch = 0
        self.shape = None
        torch.cuda.synchronize(device)
        dist.barrier(group=ep.group)

    def ensure(self, n_slots: int, H: int):
        if self.shape == (n_slots, H):
            return
        from . import symm

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.ep.group)   # nobody still stores into the buffers that are about to be replaced
        El = self.ep.local_experts
        self.cap = (int(self.capacity * n_slots) + 127) // 128 * 128 + El * 128
        self.rows = symm.symmetric_zeros(self.cap * H, torch.bfloat16, self.device, self.ep.group)
        self.src = symm.symmetric_zeros(self.cap, torch.int32, self.device, self.ep.group)
        self.back = symm.symmetric_zeros(n_slots * H, torch.bfloat16, self.device, self.ep.group)
        self.rows_ptrs, self.src_ptrs, self.back_ptrs = symm.peer_ptrs(self.rows), symm.peer_ptrs(self.src), symm.peer_ptrs(self.back)
        self.identity = torch.arange(n_slots, dtype=torch.int32, device=self.device)
        self.shape = (n_slots, H)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.ep.group)

    def exchange(self):
        """Everything this rank stored into peer memory so far is visible to a peer once it passes this point, and vice
        versa: signal, then a bounded device-side wait for every other rank's signal."""
        from ..ops import cuda as cu

        self.epoch += 1
        cu._C.signal_peers_at(self.flag_ptrs, 0, self.ep.rank, self.epoch)
        cu._C.wait_flags(self.flags.data_ptr(), 0, self.ep.size, self.epoch, self.ep.rank)
        cu._tick(2)


class _EPPlan:
    """Routing of one layer under the fused transport: ``dest[slot]`` = row of the slot inside its owner's buffer."""

    def __init__(self, experts, fused: EPFused, k: int):
        from ..ops import cuda as cu

        ep = fused.ep
        self.fused, self.k = fused, k
        self.flat = experts.reshape(-1).to(torch.int32).contiguous()
        self.n_slots = self.flat.numel()
        hist, counts, prefix = cu._C.moe_plan_count(self.flat, ep.n_experts)
        cu._C.ep_push_counts(counts, fused.counts_ptrs, ep.rank)
        fused.exchange()
        self.row_base, self.prefix_local, self.tot_local = cu._C.ep_plan(fused.counts, ep.size, ep.rank, fused.cap)
        self.dest = cu._C.moe_plan_place_remote(self.flat, hist, prefix, self.row_base, fused.cap)
        self.src_of_row = None
        cu._tick(5)

    def dispatch(self, src, scale):
        """Rows of ``src [T, H]`` (times ``scale[slot]``) to the owners of their slots' experts; returns what THIS rank
        received as a private ``[cap, H]`` tensor (padding rows zero) — the symmetric buffer is free for the next use."""
        from ..ops import cuda as cu

        f, ep = self.fused, self.fused.ep
        H = src.shape[1]
        cu._C.ep_dispatch(src.contiguous(), self.flat, self.dest, scale, self.k, ep.local_experts, ep.rank, f.rows_ptrs, f.src_ptrs)
        f.exchange()
        rows = f.rows.view(f.cap, H)
        cu._C.ep_zero_padding(rows, f.src, self.prefix_local, self.tot_local)
        cu._tick(2)
        if self.src_of_row is None:
            self.src_of_row = f.src.clone()
        return rows.clone()

    def collect(self, rows_local):
        """Rows this rank computed, back to the slots they came from; returns ``[n_slots, H]`` (private copy)."""
        from ..ops import cuda as cu

        f = self.fused
        cu._C.ep_return(rows_local.contiguous(), self.src_of_row, self.prefix_local, self.n_slots, f.back_ptrs)
        f.exchange()
        cu._tick()
        return f.back.view(self.n_slots, rows_local.shape[1]).clone()


class _EPDispatch(torch.autograd.Function):
    @staticmethod
    def forward(fctx, x, plan):
        fctx.plan, fctx.T = plan, x.shape[0]
        return plan.dispatch(x, None)

    @staticmethod
    def backward(fctx, drows):
        from ..ops import cuda as cu

        plan = fctx.plan
        back = plan.collect(drows)
        dx, _ = cu._C.moe_tokens_from_rows(back, plan.fused.identity, None, fctx.T, plan.k, True, None)
        cu._tick()
        return dx, None


class _EPCombine(torch.autograd.Function):
    @staticmethod
    def forward(fctx, y, w, plan):
        from ..ops import cuda as cu

        T = w.shape[0]
        wf = w.float().contiguous()
        back = plan.collect(y)
        fctx.plan, fctx.w_dtype = plan, w.dtype
        fctx.save_for_backward(back, wf)
        out, _ = cu._C.moe_tokens_from_rows(back, plan.fused.identity, wf, T, plan.k, True, None)
        cu._tick()
        return out

    @staticmethod
    def backward(fctx, dout):
        from ..ops import cuda as cu

        back, wf = fctx.saved_tensors
        plan = fctx.plan
        dout = dout.contiguous()
        _, dw = cu._C.moe_tokens_from_rows(back, plan.fused.identity, None, wf.shape[0], plan.k, False, dout)
        cu._tick()
        dy = plan.dispatch(dout, wf.reshape(-1))
        return dy, dw.to(fctx.w_dtype), None


def _ep_moe_experts_fused(x, gate_up_local, down_local, weights, experts, ep: EPContext):
    from ..ops import cuda as cu
    from ..ops.moe_cuda import _GroupedLinear

    T, H = x.shape
    k = experts.shape[1]
    ep.fused.ensure(T * k, H)
    plan = _EPPlan(experts, ep.fused, k)
    xs = _EPDispatch.apply(x, plan)
    h = _GroupedLinear.apply(xs, gate_up_local, plan.prefix_local)
    y = _GroupedLinear.apply(cu.swiglu(h), down_local, plan.prefix_local)
    return _EPCombine.apply(y, weights, plan)


def ep_moe_experts(x, gate_up_local, down_local, weights, experts, ep: EPContext):
    """``x [T,H]``; ``gate_up_local [E/ep, 2I, H]``, ``down_local [E/ep, H, I]``; ``weights`` / ``experts`` ``[T,k]``
    with global expert ids.  Returns ``sum_j w[t,j] * expert_{e[t,j]}(x_t)`` like ``ops.moe_experts``."""
    from .. import ops

    if ep.fused is not None and x.is_cuda and x.dtype == torch.bfloat16:
        from ..ops.moe_cuda import grouped_usable

        if grouped_usable(x, gate_up_local, down_local):
            return _ep_moe_experts_fused(x, gate_up_local, down_local, weights, experts, ep)

    T, H = x.shape
    k = experts.shape[1]
    El = ep.local_experts
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)               # pairs sorted by expert id = by owner rank, then expert
    tok_of_pair = (order // k)
    # how many pairs go to each rank / expert: one small exchange of the [ep, E_local] count matrix
    counts = torch.bincount(flat_e, minlength=ep.n_experts).reshape(ep.size, El)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=ep.group)   # row s: pairs from source rank s per local expert
    both = torch.stack((counts.sum(1), recv_counts.sum(1))).tolist()   # the one host read of this layer
    in_splits, out_splits = [int(v) for v in both[0]], [int(v) for v in both[1]]
    sent = x.index_select(0, tok_of_pair)
    recv = _AllToAllRows.apply(sent, in_splits, out_splits, ep.group)
    # rows arrive source-major with each source's rows sorted by local expert
    local_e = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(ep.size), recv_counts.reshape(-1),
                                      output_size=sum(out_splits))
    if recv.shape[0]:
        y = ops.moe_experts(recv, gate_up_local, down_local, torch.ones(recv.shape[0], 1, dtype=x.dtype, device=x.device),
                            local_e.reshape(-1, 1))
    else:
        y = recv + 0.0 * (gate_up_local.sum() + down_local.sum()).to(recv.dtype)  # keeps the parameters in the graph
    back = _AllToAllRows.apply(y, out_splits, in_splits, ep.group)          # back in `order`
    # weighted combine in slot order: pair (t, j) sits at inverse[t * k + j]
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device)
    per_slot = back.index_select(0, inverse).reshape(T, k, H)
    return (per_slot.float() * weights.reshape(T, k, 1).float()).sum(1).to(x.dtype)


def _shard_hooks(mod, ep: EPContext):
    """Keep ``state_dict`` / ``load_state_dict`` of an expert container in the full ``[E, ...]`` layout."""
    names = ("gate_up_proj", "down_proj")

    def post_hook(module, state, prefix, _local_metadata):
        for n in names:
            key = prefix + n
            if key in state and ep.size > 1:
                t = state[key]
                parts = [torch.empty_like(t) for _ in range(ep.size)]
                dist.all_gather(parts, t.contiguous(), group=ep.group)
                state[key] = torch.cat(parts, 0)
        return state

    def pre_hook(state, prefix, *_):
        for n in names:
            key = prefix + n
            if key in state and state[key].shape[0] == ep.n_experts and ep.size > 1:
                El = ep.local_experts
                state[key] = state[key][ep.rank * El:(ep.rank + 1) * El]

    mod._register_state_dict_hook(post_hook)
    mod._register_load_state_dict_pre_hook(pre_hook)


def apply_ep(model, mesh, ep_size: int, fused: bool = False) -> EPContext | None:
    """Shard every ``SparseMoeBlock``'s experts over groups of ``ep_size`` consecutive data-parallel ranks.
    ``fused``: tokens travel by peer stores over symmetric memory (GPUs of one NVLink domain) instead of all-to-all."""
    from ..models.layers import SparseMoeBlock

    blocks = [m for m in model.modules() if isinstance(m, SparseMoeBlock)]
    if ep_size <= 1 or not blocks:
        return None
    if not dist.is_initialized():
        raise RuntimeError("expert parallelism needs torch.distributed")
    if mesh.tp > 1:
        raise ValueError("expert parallelism is combined with data parallelism only (tp_size must be 1)")
    dp = mesh.dp
    if dp % ep_size:
        raise ValueError(f"ep_size {ep_size} must divide the data-parallel size {dp}")
    n_experts = blocks[0].n_experts
    if n_experts % ep_size:
        raise ValueError(f"{n_experts} experts do not divide over ep_size {ep_size}")
    # every rank creates every group, in the same order
    my_group = my_replica = None
    for g0 in range(0, dp, ep_size):
        ranks = list(range(g0, g0 + ep_size))
        grp = dist.new_group(ranks)
        if mesh.rank in ranks:
            my_group = grp
    n_rep = dp // ep_size
    for r in range(ep_size):
        ranks = [r + i * ep_size for i in range(n_rep)]
        grp = dist.new_group(ranks) if n_rep > 1 else None
        if mesh.rank in ranks:
            my_replica = grp
    ep = EPContext(group=my_group, size=ep_size, rank=mesh.rank % ep_size, replica_group=my_replica, replica_size=n_rep,
                   n_experts=n_experts)
    El = ep.local_experts
    for blk in blocks:
        ex = blk.experts
        for n in ("gate_up_proj", "down_proj"):
            p = getattr(ex, n)
            local = torch.nn.Parameter(p.detach()[ep.rank * El:(ep.rank + 1) * El].clone(), requires_grad=p.requires_grad)
            local._ep_sharded = True
            setattr(ex, n, local)
        _shard_hooks(ex, ep)
        blk.ep = ep
    if fused and mesh.device.type == "cuda":
        ep.fused = EPFused(ep, mesh.device)
    model._ep_ctx = ep
    return ep
