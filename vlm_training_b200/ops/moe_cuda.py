"""Routed-expert MLP on CUDA with grouped tcgen05 GEMMs: one launch per projection for ALL experts.

Slots (token, k) are sorted by expert and written into a padded buffer in which every expert owns whole 128-row tiles
(rows behind an expert's tokens are zero); a device-side prefix of tile counts tells the GEMM kernel which expert a tile
belongs to (``csrc/gemm_sm100.cu``, grouped modes).  Nothing is read back to the host: the buffer has a static capacity
(``T k`` rows plus one tile per expert), so the step stays free of device->host synchronisation, also under expert
parallelism.  Backward uses the same kernel: grouped dgrad (every expert's ``dY W``) and grouped wgrad (the contraction
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
        y = torch.zeros(x.shape[0], N, dtype=x.dtype, device=x.device)  # rows beyond the last used tile stay zero
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
            dx = torch.zeros_like(x)
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


def moe_experts_cuda(x, gate_up, down, weights, experts):
    T, H = x.shape
    E = gate_up.shape[0]
    k = experts.shape[1]
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)             # slots grouped by expert
    e_sorted = flat_e.index_select(0, order)
    tok = order // k                                         # source token of every sorted slot
    counts = torch.bincount(flat_e, minlength=E)
    tiles = (counts + (TILE - 1)) // TILE
    prefix = torch.zeros(E + 1, dtype=torch.int32, device=x.device)
    prefix[1:] = tiles.cumsum(0)
    start = counts.cumsum(0) - counts                        # first sorted slot of every expert
    dest = prefix[:-1].long().index_select(0, e_sorted) * TILE + (torch.arange(order.numel(), device=x.device)
                                                                  - start.index_select(0, e_sorted))
    cap = (T * k + TILE - 1) // TILE * TILE + E * TILE       # static upper bound of the padded rows
    ws = weights.reshape(-1).index_select(0, order).to(x.dtype)
    if not grouped_usable(x, gate_up, down):
        return _moe_experts_loop(x, gate_up, down, ws, tok, counts, T)
    xs = torch.zeros(cap, H, dtype=x.dtype, device=x.device).index_copy(0, dest, x.index_select(0, tok))
    h = _GroupedLinear.apply(xs, gate_up, prefix)
    y = _GroupedLinear.apply(cu.swiglu(h), down, prefix)
    ys = y.index_select(0, dest) * ws.unsqueeze(-1)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device).index_add_(0, tok, ys.float())
    return out.to(x.dtype)


def _moe_experts_loop(x, gate_up, down, ws, tok, counts, T):
    """One GEMM per non-empty expert (shapes the grouped kernel does not take); reads the ranges back to the host."""
    E, H = gate_up.shape[0], x.shape[1]
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
