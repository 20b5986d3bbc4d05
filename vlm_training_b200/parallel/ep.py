"""Expert parallelism for the sparse MoE block: every rank of the expert-parallel group owns ``E / ep``
consecutive experts; routed tokens travel to the owner of their expert (all-to-all dispatch), run through the
local experts as one grouped computation, and travel back (all-to-all combine), where the routing weights are
applied in a fixed slot order so the result does not depend on arrival order.

The reference has no expert parallelism (its MoE model runs every expert on every rank, reference:
models/qwen3_5/model.py:715-751); this is an addition for the 256-expert configuration.

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


def ep_moe_experts(x, gate_up_local, down_local, weights, experts, ep: EPContext):
    """``x [T,H]``; ``gate_up_local [E/ep, 2I, H]``, ``down_local [E/ep, H, I]``; ``weights`` / ``experts`` ``[T,k]``
    with global expert ids.  Returns ``sum_j w[t,j] * expert_{e[t,j]}(x_t)`` like ``ops.moe_experts``."""
    from .. import ops

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


def apply_ep(model, mesh, ep_size: int) -> EPContext | None:
    """Shard every ``SparseMoeBlock``'s experts over groups of ``ep_size`` consecutive data-parallel ranks."""
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
    model._ep_ctx = ep
    return ep
