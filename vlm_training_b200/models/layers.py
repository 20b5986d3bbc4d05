"""Decoder building blocks shared by Qwen3, Qwen3-VL and Qwen3.5.

All blocks work on ONE packed row ``x [T, H]`` plus a :class:`RowContext` that
carries everything derived from ``cu_seqlens`` (built once per batch on the
host).  Projections that the HF checkpoints store separately (q/k/v, gate/up,
the GDN in-projections) are held as ONE fused parameter so they run as one
GEMM; ``state_dict()`` still shows the HF names because the owning module
splits the fused tensor into views on save and fills it on load.

Tensor parallelism is built in: after :func:`vlm_training_b200.parallel.tp.apply_tp`
a block holds only its rank's rows/columns and its ``tp`` context tells the
forward which collectives to run.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from .. import ops
from ..parallel.tp_comm import TPContext, column_input, column_linear, row_linear, row_output
from .config import TextConfig

_NO_TP = TPContext()


@dataclass
class RowContext:
    """Per-batch metadata for one packed row (all host-built, no device syncs)."""

    cu_seqlens: torch.Tensor  # int32 [n_docs + 1] on the compute device
    max_seqlen: int
    cos: torch.Tensor | None = None  # [T, R]
    sin: torch.Tensor | None = None
    seq_idx: torch.Tensor | None = None  # int32 [T] document index (GDN conv)
    extras: dict = field(default_factory=dict)


# ----------------------------------------------------------------------------- basics
class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, offset: bool = False):
        super().__init__()
        self.eps, self.offset = eps, offset
        self.weight = nn.Parameter(torch.zeros(dim) if offset else torch.ones(dim))

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps, self.offset)


class Linear(nn.Module):
    """``y = x W^T (+ b)`` with ``W [out, in]``; ``parallel`` is one of
    None | "column" | "row" and only records how ``apply_tp`` shards it."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, parallel: str | None = None):
        super().__init__()
        self.in_features, self.out_features, self.parallel = in_features, out_features, parallel
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.tp = _NO_TP

    def forward(self, x):
        if self.parallel == "column":
            return column_linear(x, self.weight, self.bias, self.tp, site=self)
        if self.parallel == "row":
            y = row_linear(x, self.weight, self.tp)
            return y if self.bias is None else y + self.bias
        return ops.linear(x, self.weight, self.bias)


class FusedLinear(Linear):
    """Several HF ``nn.Linear`` weights stacked on the output dim.

    ``splits`` maps the HF sub-module name to its number of output rows.  The
    parent module must call :func:`expose_fused` so the state dict shows
    ``<name>.weight`` instead of ``<attr>.weight``."""

    def __init__(self, in_features: int, splits: "OrderedDict[str, int]", bias: bool = False,
                 parallel: str | None = "column"):
        super().__init__(in_features, sum(splits.values()), bias=bias, parallel=parallel)
        self.splits = OrderedDict(splits)

    def split_views(self, tensor=None):
        t = self.weight if tensor is None else tensor
        out, o = OrderedDict(), 0
        for name, n in self.splits.items():
            out[name] = t.narrow(0, o, n)
            o += n
        return out


def expose_fused(parent: nn.Module, attr: str):
    """Make ``parent.<attr>`` (a FusedLinear) appear in state dicts under the
    names of its splits, e.g. ``self_attn.q_proj.weight`` (HF key layout,
    reference: models/qwen3_vl/model.py:612-621)."""

    def save_hook(module, state, prefix, _meta):
        fused: FusedLinear = getattr(module, attr)
        for suffix in ("weight", "bias"):
            key = f"{prefix}{attr}.{suffix}"
            if key not in state:
                continue
            t = state.pop(key)
            o = 0
            for name, n in fused.splits.items():
                state[f"{prefix}{name}.{suffix}"] = t.narrow(0, o, n)
                o += n
        return state

    def load_hook(module, state, prefix, *_):
        fused: FusedLinear = getattr(module, attr)
        for suffix in ("weight", "bias"):
            if getattr(fused, suffix) is None:
                continue
            parts = [state.get(f"{prefix}{name}.{suffix}") for name in fused.splits]
            if all(p is None for p in parts):
                continue
            if any(p is None for p in parts):
                missing = [n for n, p in zip(fused.splits, parts) if p is None]
                raise KeyError(f"state dict misses {[prefix + m + '.' + suffix for m in missing]}")
            for name in fused.splits:
                state.pop(f"{prefix}{name}.{suffix}")
            state[f"{prefix}{attr}.{suffix}"] = torch.cat([p.to(parts[0].device) for p in parts], 0)

    parent._register_state_dict_hook(save_hook)
    parent._register_load_state_dict_pre_hook(load_hook, with_module=True)


# ----------------------------------------------------------------------------- MLP
class SwiGLUMLP(nn.Module):
    def __init__(self, hidden: int, intermediate: int):
        super().__init__()
        self.gate_up = FusedLinear(hidden, OrderedDict(gate_proj=intermediate, up_proj=intermediate), parallel="column")
        self.down_proj = Linear(intermediate, hidden, parallel="row")
        expose_fused(self, "gate_up")

    def forward(self, x):
        if not self.down_proj.tp.enabled:
            return ops.swiglu_linear(self.gate_up(x), self.down_proj.weight)
        return self.down_proj(ops.swiglu(self.gate_up(x)))

    def forward_prenorm(self, x, residual, norm: "RMSNorm"):
        """``r = x + residual; mlp(norm(r))`` → ``(out, r)`` with the norm fused into the gate/up projection."""
        if self.gate_up.tp.enabled:
            h, r = ops.add_rms_norm(x, residual, norm.weight, norm.eps, norm.offset)
            return self.forward(h), r
        gu, r = ops.rms_norm_linear(x, norm.weight, self.gate_up.weight, norm.eps, norm.offset, residual)
        return ops.swiglu_linear(gu, self.down_proj.weight), r


# ----------------------------------------------------------------------------- attention
class SelfAttention(nn.Module):
    """Causal varlen GQA attention with per-head QK RMSNorm and (M)RoPE; with
    ``attn_output_gate`` the q projection also emits a per-head sigmoid gate
    (reference: models/qwen3_vl/model.py:230-278, models/qwen3_5/model.py:74-136)."""

    def __init__(self, cfg: TextConfig):
        super().__init__()
        self.cfg = cfg
        D = cfg.head_dim
        self.n_q, self.n_kv, self.head_dim = cfg.num_attention_heads, cfg.num_key_value_heads, D
        self.gated = cfg.attn_output_gate
        self.qkv = FusedLinear(cfg.hidden_size, OrderedDict(
            q_proj=self.n_q * D * (2 if self.gated else 1), k_proj=self.n_kv * D, v_proj=self.n_kv * D), parallel="column")
        self.o_proj = Linear(self.n_q * D, cfg.hidden_size, parallel="row")
        self.q_norm = RMSNorm(D, cfg.rms_norm_eps, cfg.offset_norm)
        self.k_norm = RMSNorm(D, cfg.rms_norm_eps, cfg.offset_norm)
        self.scale = D ** -0.5
        expose_fused(self, "qkv")
        if cfg.dsa:
            # indexer of the sparse-attention variant: small projections that score keys
            self.idx_q = Linear(cfg.hidden_size, cfg.dsa_index_heads * cfg.dsa_index_dim)
            self.idx_k = Linear(cfg.hidden_size, cfg.dsa_index_dim)
            self.idx_w = Linear(cfg.hidden_size, cfg.dsa_index_heads)

    def forward(self, x, ctx: RowContext, prenorm: "RMSNorm | None" = None):
        """``prenorm``: apply this RMSNorm to ``x`` first, fused into the qkv projection where possible."""
        if prenorm is not None and not self.qkv.tp.enabled and not self.cfg.dsa:
            qkv = ops.rms_norm_linear(x, prenorm.weight, self.qkv.weight, prenorm.eps, prenorm.offset)
        else:
            if prenorm is not None:
                x = prenorm(x)
            qkv = self.qkv(x)
        T = qkv.shape[0]
        q, k, v, gate = ops.qkv_norm_rope(qkv, self.n_q, self.n_kv, self.head_dim, self.q_norm.weight,
                                          self.k_norm.weight, ctx.cos, ctx.sin, self.cfg.rms_norm_eps,
                                          self.cfg.offset_norm, self.gated)
        if self.cfg.dsa:
            xin = column_input(x, self.qkv.tp) if self.qkv.tp.enabled else x
            iq = self.idx_q(xin).view(T, self.cfg.dsa_index_heads, self.cfg.dsa_index_dim)
            o = ops.dsa_attention(q, k, v, iq, self.idx_k(xin), self.idx_w(xin), ctx.cu_seqlens,
                                  self.cfg.dsa_topk, self.scale, cu_host=ctx.extras.get("cu_host"))
        else:
            o = ops.attention_varlen(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, True, self.scale)
        o = o.reshape(T, self.n_q * self.head_dim)
        if gate is not None:
            o = ops.sigmoid_mul(o, gate)
        return self.o_proj(o)


# ----------------------------------------------------------------------------- gated delta net
class GatedRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x, z):
        return ops.rms_norm_gated(x, z, self.weight, self.eps)


class _DepthwiseConvWeight(nn.Module):
    """Holds ``weight [C, 1, K]`` under the HF name ``conv1d.weight``."""

    def __init__(self, channels: int, k: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(channels, 1, k))


class GatedDeltaNet(nn.Module):
    """Linear-attention mixer of Qwen3.5 (reference: models/qwen3_5/model.py:138-235).

    ``in_proj`` fuses ``in_proj_qkv | in_proj_z | in_proj_b | in_proj_a`` into
    one GEMM.  Head counts are the LOCAL ones after tensor-parallel sharding."""

    def __init__(self, cfg: TextConfig):
        super().__init__()
        self.cfg = cfg
        self.n_k, self.n_v = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.d_k, self.d_v = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.n_k * self.d_k, self.n_v * self.d_v
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.in_proj = FusedLinear(cfg.hidden_size, OrderedDict(
            in_proj_qkv=self.conv_dim, in_proj_z=self.value_dim, in_proj_b=self.n_v, in_proj_a=self.n_v), parallel="column")
        self.conv1d = _DepthwiseConvWeight(self.conv_dim, cfg.linear_conv_kernel_dim)
        self.dt_bias = nn.Parameter(torch.ones(self.n_v))
        self.A_log = nn.Parameter(torch.zeros(self.n_v))
        self.norm = GatedRMSNorm(self.d_v, cfg.rms_norm_eps)
        self.out_proj = Linear(self.value_dim, cfg.hidden_size, parallel="row")
        expose_fused(self, "in_proj")

    def forward(self, x, ctx: RowContext):
        proj = self.in_proj(x)
        T = proj.shape[0]
        qkv, z, b, a = proj.split([self.conv_dim, self.value_dim, self.n_v, self.n_v], dim=-1)
        qkv = ops.causal_conv1d_silu(qkv, self.conv1d.weight.squeeze(1), ctx.seq_idx)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q = q.reshape(T, self.n_k, self.d_k)
        k = k.reshape(T, self.n_k, self.d_k)
        v = v.reshape(T, self.n_v, self.d_v)
        if self.n_v > self.n_k:
            rep = self.n_v // self.n_k
            q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
        g, beta = ops.gdn_gates(a, b, self.A_log, self.dt_bias)
        o = ops.gated_delta_rule(q, k, v, g, beta, ctx.cu_seqlens, None, 64, cu_host=ctx.extras.get("cu_host"))
        o = self.norm(o.reshape(T * self.n_v, self.d_v), z.reshape(T * self.n_v, self.d_v))
        return self.out_proj(o.reshape(T, self.value_dim))


# ----------------------------------------------------------------------------- MoE
class _Router(nn.Module):
    def __init__(self, n_experts: int, hidden: int):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(n_experts, hidden))


class _Experts(nn.Module):
    """3-D expert weights under the HF names ``experts.gate_up_proj [E,2I,H]`` and
    ``experts.down_proj [E,H,I]`` (transformers qwen3_5_moe/modeling_qwen3_5_moe.py:715-751)."""

    def __init__(self, n_experts: int, hidden: int, inter: int):
        super().__init__()
        self.gate_up_proj = nn.Parameter(torch.empty(n_experts, 2 * inter, hidden))
        self.down_proj = nn.Parameter(torch.empty(n_experts, hidden, inter))


class SparseMoeBlock(nn.Module):
    """softmax → top-k → renormalise routing over ``num_experts`` SwiGLU experts
    plus one shared expert scaled by ``sigmoid(shared_expert_gate(x))``.

    With expert parallelism (``self.ep`` set by ``apply_ep``) each rank owns
    ``E / ep`` experts; tokens travel by all-to-all dispatch and combine."""

    def __init__(self, cfg: TextConfig):
        super().__init__()
        self.cfg = cfg
        self.top_k, self.n_experts = cfg.num_experts_per_tok, cfg.num_experts
        self.gate = _Router(cfg.num_experts, cfg.hidden_size)
        self.experts = _Experts(cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size)
        self.shared_expert = SwiGLUMLP(cfg.hidden_size, cfg.shared_expert_intermediate_size)
        self.shared_expert_gate = Linear(cfg.hidden_size, 1)
        self.ep = None  # parallel.ep.EPContext

    def forward(self, x):
        shared = self.shared_expert(x)
        logits = ops.linear(x, self.gate.weight)
        w, idx = ops.moe_router(logits, self.top_k, self.cfg.norm_topk_prob)
        if self.ep is not None and self.ep.size > 1:
            from ..parallel.ep import ep_moe_experts

            routed = ep_moe_experts(x, self.experts.gate_up_proj, self.experts.down_proj, w, idx, self.ep)
        else:
            routed = ops.moe_experts(x, self.experts.gate_up_proj, self.experts.down_proj, w.to(x.dtype), idx)
        return routed + ops.sigmoid_mul(shared, self.shared_expert_gate(x))


# ----------------------------------------------------------------------------- layer / stack
class DecoderLayer(nn.Module):
    def __init__(self, cfg: TextConfig, layer_idx: int):
        super().__init__()
        self.layer_type = cfg.layer_type(layer_idx)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.offset_norm)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.offset_norm)
        if self.layer_type == "linear_attention":
            self.linear_attn = GatedDeltaNet(cfg)
        else:
            self.self_attn = SelfAttention(cfg)
        self.mlp = SparseMoeBlock(cfg) if cfg.num_experts > 0 else SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size)

    def mixer_half(self, x, ctx: RowContext):
        """Token mixer on the normalised input (attention or Gated DeltaNet); the residual add happens in the MLP half."""
        if self.layer_type == "linear_attention":
            return self.linear_attn(self.input_layernorm(x), ctx)
        return self.self_attn(x, ctx, prenorm=self.input_layernorm)

    def mlp_half(self, h, x):
        """``r = x + h; r + mlp(norm(r))``."""
        if isinstance(self.mlp, SwiGLUMLP):
            out, x = self.mlp.forward_prenorm(h, x, self.post_attention_layernorm)
            return x + out
        h, x = ops.add_rms_norm(h, x, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps,
                                self.post_attention_layernorm.offset)
        return x + self.mlp(h)

    def forward(self, x, ctx: RowContext):
        return self.mlp_half(self.mixer_half(x, ctx), x)

    def forward_sac(self, x, ctx: RowContext):
        """Selective activation checkpointing: the mixer half runs under plain autograd, so what its ops saved (the
        projections' inputs, attention output and log-sum-exp, the scan states) stays and the expensive attention /
        recurrence is not run twice; the MLP half, whose ``[T, 2 I]`` activations are the largest tensors of the
        layer, is recomputed in backward (the reference's ``sac`` keeps matmul outputs and recomputes the elementwise
        work, reference: train/infra.py:161-170,222-223; here the custom ops already decide what they keep, so the
        split is by sub-block)."""
        from torch.utils.checkpoint import checkpoint

        h = self.mixer_half(x, ctx)
        return checkpoint(self.mlp_half, h, x, use_reentrant=False)


class Decoder(nn.Module):
    """``embed_tokens`` + layers + final norm; HF names ``embed_tokens``, ``layers.N``, ``norm``.

    ``deepstack`` (Qwen3-VL): a list of ``(row_index, features)``; entry ``i`` is
    added to the hidden state at ``row_index`` after layer ``i``
    (reference: models/qwen3_vl/model.py:315-334)."""

    def __init__(self, cfg: TextConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([DecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.offset_norm)
        self.ac_mode = "off"

    def run_layers(self, x, ctx: RowContext, deepstack=None):
        for i, layer in enumerate(self.layers):
            if self.ac_mode != "off" and torch.is_grad_enabled():
                from ..parallel.ac import checkpoint_layer

                x = checkpoint_layer(layer, x, ctx, self.ac_mode)
            else:
                x = layer(x, ctx)
            if deepstack is not None and i < len(deepstack):
                idx, feats = deepstack[i]
                if idx.numel():
                    x = ops.add_rows(x, idx, feats)
        return self.norm(x)
