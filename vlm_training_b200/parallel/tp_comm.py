"""Differentiable tensor-parallel collectives on packed rows ``[T, H]``.

The tensor-parallel design is Megatron-style with sequence parallelism: between
blocks the hidden state is sharded over tokens (``[T/tp, H]``), column-parallel
projections all-gather it, row-parallel projections reduce-scatter their
partial sums back to token shards.  Without sequence parallelism the hidden
state stays replicated and the pair becomes identity / all-reduce — the layout
the reference uses (reference: train/infra.py:391-401,438-458).

Each function is an autograd ``Function`` whose backward is the conjugate
collective.  ``TPContext.backend`` selects how the bytes move: ``"dist"``
(torch.distributed: NCCL on GPUs, gloo on CPU) or ``"fused"`` (the one-kernel
NVLink paths in :mod:`vlm_training_b200.parallel.fused`), which handle the
collective inside the adjacent GEMM and bypass these functions.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class TPContext:
    group: object = None
    size: int = 1
    rank: int = 0
    sequence_parallel: bool = False
    backend: str = "dist"

    @property
    def enabled(self) -> bool:
        return self.size > 1


def _all_gather_rows(x, ctx: TPContext):
    x = x.contiguous()
    out = x.new_empty((x.shape[0] * ctx.size,) + tuple(x.shape[1:]))
    dist.all_gather_into_tensor(out, x, group=ctx.group)
    return out


def _reduce_scatter_rows(x, ctx: TPContext):
    x = x.contiguous()
    assert x.shape[0] % ctx.size == 0, "token count must divide by the tensor-parallel size"
    out = x.new_empty((x.shape[0] // ctx.size,) + tuple(x.shape[1:]))
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x, group=ctx.group)
    else:  # gloo has no reduce-scatter: all-reduce and keep the local rows
        tmp = x.clone()
        dist.all_reduce(tmp, group=ctx.group)
        n = out.shape[0]
        out.copy_(tmp[ctx.rank * n:(ctx.rank + 1) * n])
    return out


class _GatherRows(torch.autograd.Function):
    """forward all-gather along tokens; backward reduce-scatter."""

    @staticmethod
    def forward(fctx, x, ctx):
        fctx.tp = ctx
        return _all_gather_rows(x, ctx)

    @staticmethod
    def backward(fctx, g):
        return _reduce_scatter_rows(g, fctx.tp), None


class _ScatterReduceRows(torch.autograd.Function):
    """forward reduce-scatter along tokens; backward all-gather."""

    @staticmethod
    def forward(fctx, x, ctx):
        fctx.tp = ctx
        return _reduce_scatter_rows(x, ctx)

    @staticmethod
    def backward(fctx, g):
        return _all_gather_rows(g, fctx.tp), None


class _CopyToTP(torch.autograd.Function):
    """forward identity; backward all-reduce (input of a column-parallel layer)."""

    @staticmethod
    def forward(fctx, x, ctx):
        fctx.tp = ctx
        return x

    @staticmethod
    def backward(fctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=fctx.tp.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """forward all-reduce; backward identity (output of a row-parallel layer)."""

    @staticmethod
    def forward(fctx, x, ctx):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=ctx.group)
        return x

    @staticmethod
    def backward(fctx, g):
        return g, None


class _SliceRows(torch.autograd.Function):
    """forward keep this rank's token shard of a replicated tensor; backward
    all-gather (used where a replicated tensor enters the sequence-parallel region)."""

    @staticmethod
    def forward(fctx, x, ctx):
        fctx.tp = ctx
        n = x.shape[0] // ctx.size
        return x[ctx.rank * n:(ctx.rank + 1) * n].contiguous()

    @staticmethod
    def backward(fctx, g):
        return _all_gather_rows(g, fctx.tp), None


def column_input(x, ctx: TPContext):
    if not ctx.enabled:
        return x
    return _GatherRows.apply(x, ctx) if ctx.sequence_parallel else _CopyToTP.apply(x, ctx)


def row_output(y, ctx: TPContext):
    if not ctx.enabled:
        return y
    return _ScatterReduceRows.apply(y, ctx) if ctx.sequence_parallel else _ReduceFromTP.apply(y, ctx)


def gather_rows(x, ctx: TPContext):
    return _GatherRows.apply(x, ctx) if ctx.enabled else x


def slice_rows(x, ctx: TPContext):
    return _SliceRows.apply(x, ctx) if ctx.enabled else x


class _GatherUneven(torch.autograd.Function):
    """All-gather row blocks of different sizes (sizes known on every rank): forward pads each rank's block to the
    largest size, gathers, and drops the padding; backward sums every rank's gradient for the local block
    (reduce-scatter on the padded layout).  Used to share vision features produced image-parallel across the
    tensor-parallel group."""

    @staticmethod
    def forward(fctx, x, sizes, ctx, grad_identical=False):
        fctx.tp, fctx.sizes, fctx.grad_identical = ctx, sizes, grad_identical
        mx = max(sizes)
        pad = x.new_zeros((mx,) + tuple(x.shape[1:]))
        pad[: x.shape[0]].copy_(x)
        out = x.new_empty((mx * ctx.size,) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, pad, group=ctx.group)
        parts = [out[r * mx: r * mx + sizes[r]] for r in range(ctx.size)]
        return torch.cat(parts, 0)

    @staticmethod
    def backward(fctx, g):
        ctx, sizes = fctx.tp, fctx.sizes
        if fctx.grad_identical:
            # every rank already holds the complete gradient (replicated consumers): keep the local block
            o = sum(sizes[: ctx.rank])
            return g[o:o + sizes[ctx.rank]].contiguous(), None, None, None
        mx = max(sizes)
        padded = g.new_zeros((mx * ctx.size,) + tuple(g.shape[1:]))
        o = 0
        for r, n in enumerate(sizes):
            padded[r * mx: r * mx + n].copy_(g[o:o + n])
            o += n
        mine = _reduce_scatter_rows(padded, ctx)
        return mine[: sizes[ctx.rank]].contiguous(), None, None, None


def gather_uneven(x, sizes, ctx: TPContext, grad_identical: bool = False):
    """``grad_identical``: the consumers of the gathered tensor are replicated over the group, so each rank's
    gradient is already the full one (no sum in backward)."""
    return _GatherUneven.apply(x, list(sizes), ctx, grad_identical) if ctx.enabled else x
