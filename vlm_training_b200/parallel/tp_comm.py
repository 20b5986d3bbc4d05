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
NVLink paths of :mod:`vlm_training_b200.parallel.p2p`), which handle the
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
    p2p: object = None  # parallel.p2p.P2PComm when the layer collectives run as our own NVLink kernels

    @property
    def enabled(self) -> bool:
        return self.size > 1


def _all_gather_rows(x, ctx: TPContext):
    if ctx.p2p is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
        return ctx.p2p.all_gather_rows(x)
    x = x.contiguous()
    out = x.new_empty((x.shape[0] * ctx.size,) + tuple(x.shape[1:]))
    dist.all_gather_into_tensor(out, x, group=ctx.group)
    return out


def _reduce_scatter_rows(x, ctx: TPContext):
    if ctx.p2p is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % (8 * ctx.size) == 0 \
            and x.shape[0] % ctx.size == 0:
        return ctx.p2p.reduce_scatter_rows(x)
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
        out = _all_gather_rows(pad, ctx)
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


def _row_blocks(rank: int, size: int, rows: int):
    """Row ranges of the other ranks' blocks (at most two contiguous ranges) and of this rank's block."""
    others = []
    if rank > 0:
        others.append((0, rank * rows))
    if rank < size - 1:
        others.append(((rank + 1) * rows, size * rows))
    return others, (rank * rows, (rank + 1) * rows)


def _gathered_gemm(x_local, w, ctx, b_mn=False, site=None):
    """``all_gather_rows(x_local) @ op(w)``; returns ``(y_full, x_full)``.  One kernel where the shapes allow it (the
    all-gather runs inside the GEMM, :meth:`P2PComm.gemm_all_gather`); otherwise the gather is a peer pull on a side
    stream that overlaps the product of this rank's own rows."""
    from ..ops import cuda as cu

    if ctx.p2p.gemm_ag_usable(x_local, w, b_mn):
        return ctx.p2p.gemm_all_gather(x_local, w, b_mn=b_mn, site=site)
    R = x_local.shape[0]
    x_full, done = ctx.p2p.all_gather_rows_async(x_local)
    others, (o0, o1) = _row_blocks(ctx.rank, ctx.size, R)
    n_out = w.shape[1] if b_mn else w.shape[0]
    y = x_local.new_empty((R * ctx.size, n_out))
    cu._gemm(x_local, w, b_mn=b_mn, out=y[o0:o1])
    torch.cuda.current_stream().wait_event(done)
    for a, b in others:
        cu._gemm(x_full[a:b], w, b_mn=b_mn, out=y[a:b])
    return y, x_full


class _GatherLinear(torch.autograd.Function):
    """Column-parallel linear on a sequence-parallel input: ``all_gather_rows(x) @ w.T`` with the collectives overlapped.
    Forward: own rows first while the peers' rows arrive.  Backward: the input-gradient blocks that belong to the other
    ranks are computed first and announced, the own block and the weight gradient follow, and the reduce-scatter
    completes at the end, when the peers' blocks have long been written."""

    @staticmethod
    def forward(fctx, x, w, ctx, site=None):
        from ..ops import cuda as cu

        y, x_full = _gathered_gemm(x, w, ctx, site=site)
        fctx.tp = ctx
        fctx.w_param = cu._grad_target(w)
        fctx.save_for_backward(x_full, w)
        return y

    @staticmethod
    def backward(fctx, dy):
        from ..ops import cuda as cu

        ctx = fctx.tp
        x_full, w = fctx.saved_tensors
        dy = dy.contiguous()
        T, K = x_full.shape
        dx = None
        if fctx.needs_input_grad[0]:
            if ctx.p2p.gemm_rs_usable(dy, w) and K % 8 == 0:
                # input gradient with the reduce-scatter inside the GEMM: the epilogue stores every row block into its
                # owner's memory while the remaining tiles are computed; the final sum reads local memory only
                dx = ctx.p2p.gemm_reduce_scatter(dy, w, b_mn=True)
            else:
                buf, handle = ctx.p2p.reduce_scatter_begin(T, K)
                others, (o0, o1) = _row_blocks(ctx.rank, ctx.size, T // ctx.size)
                for a, b in others:
                    cu._gemm(dy[a:b], w, b_mn=True, out=buf[a:b])
                handle.signal()
                cu._gemm(dy[o0:o1], w, b_mn=True, out=buf[o0:o1])
        dw = cu._wgrad(dy, x_full, fctx.w_param) if fctx.needs_input_grad[1] else None
        if fctx.needs_input_grad[0] and dx is None:
            dx = handle.result(dy)
        return dx, dw, None, None


def gather_linear_usable(x, weight, bias, ctx: TPContext) -> bool:
    return (ctx.enabled and ctx.sequence_parallel and ctx.p2p is not None and bias is None and x.is_cuda
            and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous() and x.shape[0] % 128 == 0
            and x.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0)


def column_linear(x, weight, bias, ctx: TPContext, site=None):
    """``linear(column_input(x), weight, bias)``; on the peer-to-peer backend with sequence parallelism the all-gather
    runs inside the GEMM kernel.  ``site``: the calling module; its gathered input is kept in a persistent symmetric
    buffer of that site for the backward pass."""
    if not getattr(weight, "_vlmt_fp8", False) and gather_linear_usable(x, weight, bias, ctx):   # FP8 linears: plain collectives
        return _GatherLinear.apply(x, weight, ctx, site)
    from .. import ops

    return ops.linear(column_input(x, ctx), weight, bias)


class _RowLinearReduceScatter(torch.autograd.Function):
    """Row-parallel linear whose reduce-scatter is fused into the GEMM epilogue (sequence-parallel output
    ``[T/tp, out]``).  Backward: all-gather ``dy`` (peer pull), then the usual dgrad / wgrad GEMMs."""

    @staticmethod
    def forward(fctx, x, w, ctx):
        from ..ops import cuda as cu

        fctx.tp = ctx
        fctx.w_param = cu._grad_target(w)
        fctx.save_for_backward(x, w)
        return ctx.p2p.gemm_reduce_scatter(x, w)

    @staticmethod
    def backward(fctx, dy):
        from ..ops import cuda as cu

        x, w = fctx.saved_tensors
        if fctx.needs_input_grad[0]:
            dx, dy_full = _gathered_gemm(dy.contiguous(), w, fctx.tp, b_mn=True)   # gather overlapped with the own rows
        else:
            dx, dy_full = None, _all_gather_rows(dy.contiguous(), fctx.tp)
        dw = cu._wgrad(dy_full, x, fctx.w_param) if fctx.needs_input_grad[1] else None
        return dx, dw, None


def row_linear(x, weight, ctx: TPContext):
    """``row_output(linear(x, weight))``; on the peer-to-peer backend with sequence parallelism the collective runs
    inside the GEMM kernel's epilogue."""
    if (ctx.enabled and ctx.sequence_parallel and ctx.p2p is not None and not getattr(weight, "_vlmt_fp8", False)
            and ctx.p2p.gemm_rs_usable(x, weight)):
        return _RowLinearReduceScatter.apply(x, weight, ctx)
    from .. import ops

    return row_output(ops.linear(x, weight, None), ctx)
