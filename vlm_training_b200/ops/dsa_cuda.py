"""DSA sparse attention on CUDA.

Indexer scores -> per-query top-k key selection -> attention restricted to the selected keys, per document and in query
blocks of 1024 so the score matrix is never larger than ``block x L``.  The documents and blocks are walked from the host
copy of the boundaries (no device read).  Per block:

* selection: ``csrc/dsa_indexer_sm100.cu`` (indexer heads' products on the tensor cores folded into fp32 scores, then a
  radix-select top-k; -1 in unused slots) for 4 indexer heads of 64 channels in bf16, else ``einsum`` / ``topk`` under
  ``no_grad`` — the selection is an index set, nothing of it is kept for backward;
* attention over the selected keys: the tcgen05 kernels of ``csrc/dsa_attention_sm100.cu`` (head size 256, 8 query heads
  per kv head), else the CUDA-core kernels of ``csrc/dsa_attention.cu`` (one CTA per query and kv head reads each selected
  key / value row once for the query heads that share it), else a gathered dense softmax of tensor operations.

Documents no longer than ``topk`` take the dense tcgen05 attention kernel directly (the selection keeps every causal key).
"""
from __future__ import annotations

import math
import os

import torch
import torch.utils.checkpoint as _ckpt

from . import cuda as cu

_QBLOCK = 1024


class _SelectedAttention(torch.autograd.Function):
    """Attention of a query block over per-query key lists, as the CUDA kernels of ``csrc/dsa_attention.cu``.
    ``sel`` is int32 ``[B, kk]`` with -1 in unused slots.  The key / value gradients of the whole document come back as
    float32 (atomics accumulate them), autograd sums the blocks' contributions."""

    @staticmethod
    def forward(ctx, qb, kd, vd, sel, scale):
        qb, kd, vd = qb.contiguous(), kd.contiguous(), vd.contiguous()
        o, lse = cu._C.dsa_fwd(qb, kd, vd, sel, scale, os.environ.get("VLMT_DSA_TC", "1") != "0")
        cu._tick()
        ctx.save_for_backward(qb, kd, vd, sel, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        qb, kd, vd, sel, o, lse = ctx.saved_tensors
        dk = torch.zeros(kd.shape, dtype=torch.float32, device=kd.device)
        dv = torch.zeros(vd.shape, dtype=torch.float32, device=vd.device)
        dq = cu._C.dsa_bwd(d_o.contiguous(), qb, kd, vd, sel, o, lse, dk, dv, ctx.scale, os.environ.get("VLMT_DSA_TC", "1") != "0")
        cu._tick()
        return dq.to(qb.dtype), dk.to(kd.dtype), dv.to(vd.dtype), None, None


def _native(q, k) -> bool:
    return (hasattr(cu._C, "dsa_fwd") and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
            and cu._C.dsa_supported(q.shape[-1], q.shape[1] // k.shape[1]) and os.environ.get("VLMT_DSA_NATIVE", "1") != "0")


def _block_attention(qb, kd, vd, sel, valid, scale, rep):
    """Softmax attention of one query block over its selected keys: ``qb [B,Hq,D]``, ``kd, vd [L,Hkv,D]``,
    ``sel, valid [B,kk]``.  Differentiable with respect to ``qb``, ``kd`` and ``vd``."""
    B, Hq, D = qb.shape
    Hkv = kd.shape[1]
    # head-major float32 copies of the document's keys / values (small), gathered straight into the [Hkv, B, kk, D]
    # layout the batched products want: one write of the gathered block, no permuted re-copies
    kt = kd.float().transpose(0, 1).contiguous()
    vt = vd.float().transpose(0, 1).contiguous()
    kg = kt[:, sel]                                             # [Hkv, B, kk, D]
    vg = vt[:, sel]
    q4 = qb.float().view(B, Hkv, rep, D).transpose(0, 1)         # [Hkv, B, rep, D]
    att = torch.matmul(q4, kg.transpose(-1, -2)) * scale         # [Hkv, B, rep, kk]
    att = att.masked_fill(~valid[None, :, None, :], float("-inf")).softmax(-1)
    out = torch.matmul(att, vg)                                  # [Hkv, B, rep, D]
    return out.transpose(0, 1).reshape(B, Hq, D)


def _native_indexer(idx_q, idx_k) -> bool:
    return (hasattr(cu._C, "dsa_select") and idx_q.dtype == torch.bfloat16 and idx_k.dtype == torch.bfloat16 and idx_q.dim() == 3
            and idx_q.shape[1:] == (4, 64) and idx_k.shape[-1] == 64 and os.environ.get("VLMT_DSA_INDEXER", "1") != "0")


def dsa_attention_cuda(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk, scale=None, cu_host=None):
    """``cu_host``: the document boundaries as a host sequence (saves the device read of ``cu_seqlens``)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    bounds = [int(x) for x in cu_host] if cu_host is not None else cu_seqlens.tolist()
    native = _native(q, k)
    fused_select = native and _native_indexer(idx_q, idx_k)
    if fused_select:
        with torch.no_grad():
            iq_c, ik_c, iw_c = idx_q.contiguous(), idx_k.contiguous(), idx_w.float().contiguous()
    if max(b - a for a, b in zip(bounds[:-1], bounds[1:])) <= topk:
        return cu.attention_varlen(q, k, v, cu_seqlens, 0, True, scale)
    # documents end where the packed row ends: tokens behind the last boundary are padding
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
        ik = None if fused_select else idx_k[s:e].float()
        doc_out = []
        for b0 in range(0, L, _QBLOCK):
            b1 = min(L, b0 + _QBLOCK)
            n_keys = b1  # causal: keys [0, b1)
            if fused_select:
                # scores on the tensor cores and a radix-select top-k, two launches per block, -1 in unused slots
                sel32 = cu._C.dsa_select(iq_c, ik_c, iw_c, s + b0, b0, s, b1 - b0, min(topk, n_keys))
                cu._tick(2)
                doc_out.append(_SelectedAttention.apply(q[s + b0:s + b1], kd, vd, sel32, scale))
                continue
            with torch.no_grad():  # the selection is an index set: nothing of it is kept for backward
                sc = torch.einsum("thd,sd->ths", idx_q[s + b0:s + b1].float(), ik[:n_keys]).relu_()
                sc = (sc * idx_w[s + b0:s + b1].float().unsqueeze(-1)).sum(1)  # [B, n_keys]
                qpos = torch.arange(b0, b1, device=q.device).unsqueeze(1)
                kpos = torch.arange(n_keys, device=q.device).unsqueeze(0)
                sc = sc.masked_fill(kpos > qpos, float("-inf"))
                kk = min(topk, n_keys)
                sel = sc.topk(kk, dim=-1).indices  # [B, kk]
                valid = sel <= qpos  # picks that were -inf (fewer than kk causal keys) are masked out
                del sc
            # the gathered keys / values of a block are 2 x B x kk x Hkv x D floats (gigabytes at topk 2048): they are
            # rebuilt in backward instead of being kept, so a long document costs one block of them at a time
            if native:
                sel32 = torch.where(valid, sel, -1).to(torch.int32)
                doc_out.append(_SelectedAttention.apply(q[s + b0:s + b1], kd, vd, sel32, scale))
            else:
                doc_out.append(_ckpt.checkpoint(_block_attention, q[s + b0:s + b1], kd, vd, sel, valid, scale, rep,
                                                use_reentrant=False))
        outs.append(torch.cat(doc_out, 0).to(q.dtype))
    if bounds[-1] < T:
        outs.append(q.new_zeros(T - bounds[-1], Hq, D))
    return torch.cat(outs, 0)
