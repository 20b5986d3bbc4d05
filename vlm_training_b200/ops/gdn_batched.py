"""Gated delta rule over a packed row, batched across documents and chunks.

Same maths as :func:`vlm_training_b200.ops.reference.gated_delta_rule` (WY / UT chunk form, chunk 64,
state reset at every document boundary), restructured so the device sees few, large operations:

* tokens are scattered into a padded ``[n_chunks_total, 64]`` layout built from ``cu_seqlens`` on the host
  (padding rows have k = v = beta = g = 0 and therefore no effect);
* everything inside a chunk — decay matrices, the 64x64 triangular solve, ``w``, ``u``, the local
  attention term — runs once for all chunks of all documents and heads;
* the only sequential part is the state recurrence over chunk positions; documents are sorted by length
  so the documents still alive at chunk position ``c`` form a prefix and one batched step serves them all.

It is differentiable through autograd and is what CUDA tensors use until the dedicated recurrence kernel
lands; it needs the document lengths on the host (``cu_host``) to avoid a device sync.
"""
from __future__ import annotations

import numpy as np
import torch

from .reference import l2norm


def _layout(cu_host, chunk: int):
    cu = np.asarray(cu_host, dtype=np.int64)
    lens = np.diff(cu)
    order = np.argsort(-lens, kind="stable")  # longest document first
    n_chunks = (lens + chunk - 1) // chunk
    doc_first_chunk = np.zeros(len(lens), dtype=np.int64)
    # chunk slots are laid out chunk-position-major: slot(c, rank r of doc in `order`) so that the documents
    # alive at position c occupy a contiguous block
    max_c = int(n_chunks.max()) if len(n_chunks) else 0
    alive = [(n_chunks[order] > c).sum() for c in range(max_c)]
    base = np.concatenate(([0], np.cumsum(alive)))
    rank_of = np.empty(len(lens), dtype=np.int64)
    rank_of[order] = np.arange(len(lens))
    T = int(cu[-1])
    tok = np.arange(T)
    doc = np.searchsorted(cu[1:], tok, side="right")
    pos = tok - cu[doc]
    c = pos // chunk
    slot = base[c] + rank_of[doc]
    dst = slot * chunk + (pos % chunk)
    return dst, int(base[-1]), alive, base


def gated_delta_rule_batched(q, k, v, g, beta, cu_host, scale=None, chunk: int = 64):
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    dev = q.device
    scale = scale if scale is not None else Dk ** -0.5
    dst_np, n_slots, alive, base = _layout(cu_host, chunk)
    Tc = int(np.asarray(cu_host)[-1])
    dst = torch.from_numpy(dst_np).to(dev, non_blocking=True)

    def pad(x, fill=0.0):  # [T, H, ...] -> [n_slots, chunk, H, ...] -> [n_slots, H, chunk, ...]
        out = x.new_full((n_slots * chunk,) + tuple(x.shape[1:]), fill)
        out = out.index_copy(0, dst, x[:Tc])
        out = out.view(n_slots, chunk, *x.shape[1:])
        return out.transpose(1, 2)

    qf = pad(l2norm(q) * scale)
    kf = pad(l2norm(k))
    vf = pad(v.float())
    gf = pad(g.float())        # [N, H, C]
    bf = pad(beta.float())
    gc = gf.cumsum(-1)
    kb = kf * bf.unsqueeze(-1)
    vb = vf * bf.unsqueeze(-1)
    dec = gc.unsqueeze(-1) - gc.unsqueeze(-2)  # [N, H, C, C]: gc_i - gc_j
    strict = torch.ones(chunk, chunk, dtype=torch.bool, device=dev).tril(-1)
    incl = torch.ones(chunk, chunk, dtype=torch.bool, device=dev).tril(0)
    A = (kb @ kf.transpose(-1, -2)) * dec.masked_fill(~strict, float("-inf")).exp()
    eye = torch.eye(chunk, device=dev, dtype=torch.float32)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    w = Tm @ (kb * gc.exp().unsqueeze(-1))
    u = Tm @ vb
    qk = (qf @ kf.transpose(-1, -2)) * dec.masked_fill(~incl, float("-inf")).exp()
    qg = qf * gc.exp().unsqueeze(-1)
    last = gc[..., -1]
    kdec = kf * (last.unsqueeze(-1) - gc).exp().unsqueeze(-1)
    outs = []
    S = None
    for c, n_alive in enumerate(alive):
        lo, hi = int(base[c]), int(base[c + 1])
        if S is None:
            S = torch.zeros(n_alive, H, Dk, Dv, dtype=torch.float32, device=dev)
        else:
            S = S[:n_alive]
        vnew = u[lo:hi] - w[lo:hi] @ S
        outs.append(qg[lo:hi] @ S + qk[lo:hi] @ vnew)
        S = S * last[lo:hi].exp().unsqueeze(-1).unsqueeze(-1) + kdec[lo:hi].transpose(-1, -2) @ vnew
    o = torch.cat(outs, 0)  # [n_slots, H, C, Dv]
    o = o.transpose(1, 2).reshape(n_slots * chunk, H, Dv)
    out = o.index_select(0, dst)
    if Tc < T:
        out = torch.cat((out, out.new_zeros(T - Tc, H, Dv)), 0)
    return out.to(v.dtype)
