"""Routed-expert MLP on CUDA: own routing / permutation kernels around grouped tcgen05 GEMMs (one launch per projection
for ALL experts).

``moe_router``: softmax -> top-k -> renormalise in one kernel, one warp per token (``csrc/moe_kernels.cu``), with its
own backward.  ``moe_experts``: the ``T k`` slots (token, choice) are counting-sorted by expert on the device into a
padded buffer in which every expert owns whole 128-row tiles (``plan``: deterministic, no atomics on the placement);
``dispatch`` copies each slot's token row to its row (padding rows zero); a device-side prefix of tile counts tells
the GEMM kernel which expert a tile belongs to (``csrc/gemm_sm100.cu``, grouped modes); ``combine`` sums every token's
``k`` expert rows with the routing weights in slot order.  Nothing is read back to the host: the buffer has a static
capacity (``T k`` rows plus one tile per expert), so the step stays free of device->host synchronisation.  Backward uses the same kernel: grouped dgrad (every expert's ``dY W``) and grouped wgrad (the contraction
over an expert's rows, one ``[out, in]`` block per expert).
"""
from __future__ import annotations

import torch

from . import cuda as cu

TILE = 128


class _GroupedLinear(torch.autograd.Function):
    """``y[rows of expert e] = x[rows of expert e] @ w[e].T`` on the padded row layout; ``w [E, N, K]``."""

    @staticmethod
    def forward(ctx, x, w, prefix):
        E, N, K = w.shape
        x = x.contiguous()
        # every row of a used tile is written by the kernel (padding rows of a tile are zero in x, so zero in y); the rows
        # beyond the last used tile are written by nobody and read by nobody: the combine walks the slot -> row map, the
        # grouped weight gradient contracts over the groups' own rows only.  No fill of the whole capacity.
        y = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        cu._C.gemm_grouped(x, w.reshape(E * N, K), y, prefix, 1, False)
        cu._tick()
        ctx.save_for_backward(x, w, prefix)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, prefix = ctx.saved_tensors
        E, N, K = w.shape
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)   # as above: rows of unused tiles are never read
            cu._C.gemm_grouped(dy, w.reshape(E * N, K), dx, prefix, 1, True)     # dX = dY . W_e  (W_e read MN-major)
            cu._tick()
        if ctx.needs_input_grad[1]:
            dw = torch.empty(E * N, K, dtype=w.dtype, device=w.device)
            cu._C.gemm_grouped(dy, x, dw, prefix, 2, True)                        # dW_e = dY_e^T X_e
            cu._tick()
            dw = dw.view(E, N, K)
        return dx, dw, None


def grouped_usable(x, gate_up, down) -> bool:
    E, N2, H = gate_up.shape
    inter = down.shape[2]
    return (x.is_cuda and x.dtype == torch.bfloat16 and H % 8 == 0 and inter % 8 == 0
            and N2 % TILE == 0 and down.shape[1] % TILE == 0)   # grouped wgrad writes whole 128-row blocks per expert


class _Router(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, renorm):
        lc = logits.contiguous()
        w, e = cu._C.moe_route_fwd(lc, k, renorm)
        cu._tick()
        ctx.save_for_backward(lc, e, w)
        ctx.renorm = renorm
        ctx.mark_non_differentiable(e)
        return w, e

    @staticmethod
    def backward(ctx, dw, _de):
        logits, e, w = ctx.saved_tensors
        cu._tick()
        return cu._C.moe_route_bwd(logits, e, w, dw.float().contiguous(), ctx.renorm), None, None


def moe_router_cuda(logits, top_k: int, renorm: bool = True):
    """``(weights [T,k] fp32, experts [T,k] int64)`` like the reference statement; ties go to the lower expert id."""
    if logits.dim() != 2 or logits.shape[1] > 512 or top_k > 32 or logits.dtype not in (torch.bfloat16, torch.float32):
        from . import reference as ref

        return ref.moe_router(logits, top_k, renorm)
    w, e = _Router.apply(logits, int(top_k), bool(renorm))
    return w, e.long()


class MoePlan:
    """Where every slot goes in the padded row layout (all int32 device tensors, built without a host read)."""

    def __init__(self, experts, n_experts: int, k: int, cap_rows: int | None = None):
        flat = experts.reshape(-1).to(torch.int32).contiguous()
        self.k, self.E, self.n_slots = k, n_experts, flat.numel()
        self.cap = cap_rows if cap_rows is not None else (self.n_slots + TILE - 1) // TILE * TILE + n_experts * TILE
        self.counts, self.prefix, self.dest, self.slot_of_row = cu._C.moe_plan(flat, n_experts, self.cap)
        cu._tick(3)


class _Dispatch(torch.autograd.Function):
    """``rows[dest[slot]] = x[slot // k]``; backward sums a token's ``k`` row gradients."""

    @staticmethod
    def forward(ctx, x, plan):
        ctx.plan, ctx.T = plan, x.shape[0]
        cu._tick()
        return cu._C.moe_rows_from_tokens(x.contiguous(), plan.slot_of_row, plan.prefix, plan.k, None)

    @staticmethod
    def backward(ctx, drows):
        plan = ctx.plan
        cu._tick()
        dx, _ = cu._C.moe_tokens_from_rows(drows.contiguous(), plan.dest, None, ctx.T, plan.k, True, None)
        return dx, None


class _Combine(torch.autograd.Function):
    """``out[t] = sum_j w[t,j] rows[dest[t,j]]`` (fp32 accumulation, slot order)."""

    @staticmethod
    def forward(ctx, rows, w, plan):
        T = w.shape[0]
        wf = w.float().contiguous()
        rows = rows.contiguous()
        ctx.plan, ctx.w_dtype = plan, w.dtype
        ctx.save_for_backward(rows, wf)
        cu._tick()
        out, _ = cu._C.moe_tokens_from_rows(rows, plan.dest, wf, T, plan.k, True, None)
        return out

    @staticmethod
    def backward(ctx, dout):
        rows, wf = ctx.saved_tensors
        plan = ctx.plan
        dout = dout.contiguous()
        T = wf.shape[0]
        drows = cu._C.moe_rows_from_tokens(dout, plan.slot_of_row, plan.prefix, plan.k, wf.reshape(-1))
        _, dw = cu._C.moe_tokens_from_rows(rows, plan.dest, None, T, plan.k, False, dout)
        cu._tick(2)
        return drows, dw.to(ctx.w_dtype), None


def moe_experts_cuda(x, gate_up, down, weights, experts):
    T, H = x.shape
    E = gate_up.shape[0]
    k = experts.shape[1]
    if not grouped_usable(x, gate_up, down):
        return _moe_experts_loop(x, gate_up, down, weights, experts)
    if cu.debug_checks_enabled():
        cu.validate_row_indices(None, T, experts=experts, n_experts=E)
    plan = MoePlan(experts, E, k)
    xs = _Dispatch.apply(x, plan)
    h = _GroupedLinear.apply(xs, gate_up, plan.prefix)
    y = _GroupedLinear.apply(cu.swiglu(h), down, plan.prefix)
    return _Combine.apply(y, weights, plan)


def _moe_experts_loop(x, gate_up, down, weights, experts):
    """One GEMM per non-empty expert (shapes the grouped kernel does not take); reads the ranges back to the host."""
    T, H = x.shape
    E, k = gate_up.shape[0], experts.shape[1]
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // k
    counts = torch.bincount(flat_e, minlength=E)
    ws = weights.reshape(-1).index_select(0, order).to(x.dtype)
    bounds = torch.cat((counts.new_zeros(1), counts.cumsum(0))).tolist()
    xs = x.index_select(0, tok)
    out_slots = []
    for e in range(E):
        lo, hi = bounds[e], bounds[e + 1]
        if hi == lo:
            continue
        out_slots.append(cu.linear(cu.swiglu(cu.linear(xs[lo:hi], gate_up[e])), down[e]))
    ys = torch.cat(out_slots, 0) * ws.unsqueeze(-1)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device).index_add_(0, tok, ys.float())
    return out.to(x.dtype)
