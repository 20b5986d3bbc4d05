"""Tensor parallelism: shard a built model in place.

Megatron-style column/row sharding of the attention, Gated-DeltaNet and MLP
projections with head-aligned splits of the fused weights (the reference's plans:
train/infra.py:348-677), plus optional sequence parallelism: between blocks the
hidden state is sharded over tokens, so norms, residual adds, the embedding
lookup and the chunked cross-entropy run on ``T / tp`` tokens per rank.  The
reference keeps the hidden state replicated because its vision scatter and
DeepStack adds use full-sequence boolean masks (train/infra.py:391-401); here
those are index lists, which shard cleanly.

Replicated parameters (norms, embeddings, lm_head, the ViT, MoE router) are
tagged ``_tp_grad = "partial"`` (their gradient must be summed over the TP group)
or ``"identical"``; sharded ones are tagged ``_tp_sharded = True`` and carry
``_tp_shard_dim`` and ``_tp_splits`` so checkpoints can be saved as global tensors.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..models.layers import FusedLinear, GatedDeltaNet, Linear, SelfAttention, SparseMoeBlock, SwiGLUMLP
from .tp_comm import TPContext


def _shard_rows_by_splits(weight: torch.Tensor, splits: list[int], tp: int, rank: int, unit: list[int] | None = None):
    """Take this rank's 1/tp of every split (along dim 0) and concatenate them."""
    out, o = [], 0
    for n in splits:
        if n % tp:
            raise ValueError(f"split of {n} rows is not divisible by tp={tp}")
        k = n // tp
        out.append(weight.narrow(0, o + rank * k, k))
        o += n
    return torch.cat(out, 0).contiguous()


def _replace_param(module: nn.Module, name: str, new: torch.Tensor, *, sharded: bool, dim: int | None = None, splits=None):
    old = getattr(module, name)
    p = nn.Parameter(new.clone(), requires_grad=old.requires_grad)
    p._tp_sharded = sharded
    if sharded:
        p._tp_shard_dim = dim
        p._tp_splits = splits
    setattr(module, name, p)
    return p


def _column(lin: Linear, ctx: TPContext):
    splits = list(lin.splits.values()) if isinstance(lin, FusedLinear) else [lin.out_features]
    w = _shard_rows_by_splits(lin.weight.data, splits, ctx.size, ctx.rank)
    _replace_param(lin, "weight", w, sharded=True, dim=0, splits=splits)
    if lin.bias is not None:
        b = _shard_rows_by_splits(lin.bias.data, splits, ctx.size, ctx.rank)
        _replace_param(lin, "bias", b, sharded=True, dim=0, splits=splits)
    if isinstance(lin, FusedLinear):
        for k in lin.splits:
            lin.splits[k] //= ctx.size
    lin.out_features //= ctx.size
    lin.tp = ctx


def _row(lin: Linear, ctx: TPContext):
    n = lin.in_features // ctx.size
    w = lin.weight.data.narrow(1, ctx.rank * n, n).contiguous()
    _replace_param(lin, "weight", w, sharded=True, dim=1, splits=[lin.in_features])
    lin.in_features = n
    lin.tp = ctx
    if lin.bias is not None:
        lin.bias._tp_grad = "identical"


def _attention(att: SelfAttention, ctx: TPContext):
    if att.n_kv % ctx.size or att.n_q % ctx.size:
        raise ValueError(f"heads ({att.n_q} q / {att.n_kv} kv) are not divisible by tp={ctx.size}")
    _column(att.qkv, ctx)
    _row(att.o_proj, ctx)
    att.n_q //= ctx.size
    att.n_kv //= ctx.size
    for norm in (att.q_norm, att.k_norm):  # applied to local heads only: partial gradients
        norm.weight._tp_grad = "partial"
    for name in ("idx_q", "idx_k", "idx_w"):
        if hasattr(att, name):
            for p in getattr(att, name).parameters():
                p._tp_grad = "partial"


def _gdn(g: GatedDeltaNet, ctx: TPContext):
    """Head-sharded Gated DeltaNet: rank r keeps q/k heads and v heads [r*n/tp, (r+1)*n/tp) of the fused
    in-projection, the matching conv channels and per-head parameters (reference: train/infra.py:493-600)."""
    tp, r = ctx.size, ctx.rank
    if g.n_k % tp or g.n_v % tp:
        raise ValueError(f"GDN heads ({g.n_k} k / {g.n_v} v) are not divisible by tp={tp}")
    kd, vd = g.key_dim, g.value_dim
    # in_proj rows: [q | k | v | z | b | a]; the qkv split itself has three head-aligned parts
    w = g.in_proj.weight.data
    parts = [kd, kd, vd, vd, g.n_v, g.n_v]
    new_w = _shard_rows_by_splits(w, parts, tp, r)
    _replace_param(g.in_proj, "weight", new_w, sharded=True, dim=0, splits=parts)
    conv = _shard_rows_by_splits(g.conv1d.weight.data, [kd, kd, vd], tp, r)
    _replace_param(g.conv1d, "weight", conv, sharded=True, dim=0, splits=[kd, kd, vd])
    for name in ("A_log", "dt_bias"):
        t = getattr(g, name).data
        n = t.shape[0] // tp
        _replace_param(g, name, t.narrow(0, r * n, n).contiguous(), sharded=True, dim=0, splits=[t.shape[0]])
    g.n_k //= tp
    g.n_v //= tp
    g.key_dim //= tp
    g.value_dim //= tp
    g.conv_dim = 2 * g.key_dim + g.value_dim
    for k in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a"):
        g.in_proj.splits[k] //= tp
    g.in_proj.out_features //= tp
    g.in_proj.tp = ctx
    _row(g.out_proj, ctx)
    g.norm.weight._tp_grad = "partial"


def _mlp(mlp: SwiGLUMLP, ctx: TPContext):
    _column(mlp.gate_up, ctx)
    _row(mlp.down_proj, ctx)


def apply_tp(model, mesh, sequence_parallel: bool = False, backend: str = "dist"):
    """Shard ``model`` over ``mesh.tp_group`` in place.  Returns the TPContext in use."""
    if mesh.tp == 1:
        return TPContext()
    if model.config.text.tie_word_embeddings:
        raise ValueError("tensor parallelism with tied word embeddings is not supported")  # as the reference refuses
    ctx = TPContext(group=mesh.tp_group, size=mesh.tp, rank=mesh.tp_rank, sequence_parallel=sequence_parallel, backend=backend)
    if backend == "p2p":
        from .p2p import P2PComm

        ctx.p2p = P2PComm(mesh.tp_group, mesh.device)
    dec = model.decoder
    for layer in dec.layers:
        if hasattr(layer, "self_attn"):
            _attention(layer.self_attn, ctx)
        if hasattr(layer, "linear_attn"):
            _gdn(layer.linear_attn, ctx)
        if isinstance(layer.mlp, SwiGLUMLP):
            _mlp(layer.mlp, ctx)
        elif isinstance(layer.mlp, SparseMoeBlock):
            _mlp(layer.mlp.shared_expert, ctx)
    grad_kind = "partial" if sequence_parallel else "identical"
    if model.visual is not None:
        # the tower runs image-parallel over the group: each rank sees only its share of the images
        for p in model.visual.parameters():
            p._tp_grad = "partial"
    for p in model.parameters():
        if not getattr(p, "_tp_sharded", False):
            p._tp_sharded = False
            if not hasattr(p, "_tp_grad"):
                p._tp_grad = grad_kind
    model.tp = ctx
    dec.tp = ctx
    return ctx
