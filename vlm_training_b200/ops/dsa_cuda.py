"""DSA sparse attention on CUDA.

Indexer scores → per-query top-k key selection → attention restricted to the selected keys.  This build
computes the selection with batched library kernels per document (scores by one GEMM per indexer head
block, ``topk``) in query blocks so the ``[L, L]`` score matrix is never larger than ``block x L``, and
runs the attention over the selected keys as a gathered dense softmax in the same blocks.  Documents no
longer than ``topk`` take the dense tcgen05 attention kernel directly (the selection keeps every causal key).
"""
from __future__ import annotations

import math

import torch

from . import cuda as cu

_QBLOCK = 1024


def dsa_attention_cuda(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk, scale=None):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    bounds = cu_seqlens.tolist()
    if max(b - a for a, b in zip(bounds[:-1], bounds[1:])) <= topk:
        return cu.attention_varlen(q, k, v, cu_seqlens, 0, True, scale)
    outs = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        L = e - s
        if L <= 0:
            continue
        if L <= topk:
            c = torch.tensor([0, L], dtype=torch.int32, device=q.device)
            outs.append(cu.attention_varlen(q[s:e], k[s:e], v[s:e], c, L, True, scale))
            continue
        kd, vd = k[s:e], v[s:e]
        ik = idx_k[s:e].float()
        doc_out = []
        for b0 in range(0, L, _QBLOCK):
            b1 = min(L, b0 + _QBLOCK)
            n_keys = b1  # causal: keys [0, b1)
            sc = torch.einsum("thd,sd->ths", idx_q[s + b0:s + b1].float(), ik[:n_keys]).relu_()
            sc = (sc * idx_w[s + b0:s + b1].float().unsqueeze(-1)).sum(1)  # [B, n_keys]
            qpos = torch.arange(b0, b1, device=q.device).unsqueeze(1)
            kpos = torch.arange(n_keys, device=q.device).unsqueeze(0)
            sc = sc.masked_fill(kpos > qpos, float("-inf"))
            kk = min(topk, n_keys)
            sel = sc.topk(kk, dim=-1).indices  # [B, kk]
            valid = sel <= qpos  # picks that were -inf (fewer than kk causal keys) are masked out
            kg = kd[sel].float()  # [B, kk, Hkv, D]
            vg = vd[sel].float()
            qb = q[s + b0:s + b1].float().view(b1 - b0, Hkv, rep, D)
            att = torch.einsum("bgrd,bkgd->bgrk", qb, kg) * scale
            att = att.masked_fill(~valid[:, None, None, :], float("-inf")).softmax(-1)
            doc_out.append(torch.einsum("bgrk,bkgd->bgrd", att, vg).reshape(b1 - b0, Hq, D))
        outs.append(torch.cat(doc_out, 0).to(q.dtype))
    if bounds[-1] < T:
        outs.append(q.new_zeros(T - bounds[-1], Hq, D))
    return torch.cat(outs, 0)
