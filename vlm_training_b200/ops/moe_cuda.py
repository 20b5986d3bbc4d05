"""Routed-expert MLP on CUDA: sort tokens by expert once, run every expert's SwiGLU MLP on its contiguous
slice with the tcgen05 GEMM, and combine with the routing weights by one index-add.

Token permutation and the per-expert row ranges come from a single sort + bincount; the per-expert ranges
are read back to the host once per call (one small device→host copy) to launch one GEMM per non-empty
expert.  Gradients flow through the same kernels (``ops.linear`` / ``ops.swiglu`` autograd functions).
"""
from __future__ import annotations

import torch

from . import cuda as cu


def moe_experts_cuda(x, gate_up, down, weights, experts):
    T, H = x.shape
    E = gate_up.shape[0]
    k = experts.shape[1]
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)            # slots grouped by expert
    tok = order // k                                        # source token of every slot
    counts = torch.bincount(flat_e, minlength=E)
    bounds = torch.cat((counts.new_zeros(1), counts.cumsum(0))).tolist()  # host copy of the E+1 range boundaries
    xs = x.index_select(0, tok)                             # [T*k, H] gathered once
    ws = weights.reshape(-1).index_select(0, order).to(x.dtype)
    out_slots = []
    for e in range(E):
        lo, hi = bounds[e], bounds[e + 1]
        if hi == lo:
            continue
        h = cu.linear(xs[lo:hi], gate_up[e])
        out_slots.append(cu.linear(cu.swiglu(h), down[e]))
    ys = torch.cat(out_slots, 0) * ws.unsqueeze(-1)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device).index_add_(0, tok, ys.float())
    return out.to(x.dtype)
