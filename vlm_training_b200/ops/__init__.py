"""Functional hot ops.

Every function here has two implementations: a plain-PyTorch one in
:mod:`.reference` (used for CPU tensors and as the test oracle) and a
hand-written sm_100a CUDA one in :mod:`.cuda` (used for CUDA tensors).  There
is no third path: a CUDA tensor never falls back to the PyTorch statement
silently.  If the compiled extension is missing on a machine that has a GPU,
the first CUDA call raises.

Set ``VLMT_FORCE_REFERENCE=1`` to run the PyTorch statements on CUDA tensors
(for A/B numerics only; it is slow and is never the default).
"""
from __future__ import annotations

import os

import torch

from . import reference as ref

_FORCE_REF = os.environ.get("VLMT_FORCE_REFERENCE", "0") == "1"


def _use_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_REF


def _cu():
    from . import cuda as cu  # deferred: importing it loads the extension

    return cu


# --- norms -------------------------------------------------------------------
def rms_norm(x, weight, eps: float = 1e-6, offset: bool = False):
    if _use_cuda(x):
        return _cu().rms_norm(x, weight, eps, offset)
    return ref.rms_norm(x, weight, eps, offset)


def add_rms_norm(x, residual, weight, eps: float = 1e-6, offset: bool = False):
    """``r = x + residual; y = rms_norm(r)``; returns ``(y, r)`` in one pass."""
    if _use_cuda(x):
        return _cu().add_rms_norm(x, residual, weight, eps, offset)
    r = x + residual
    return ref.rms_norm(r, weight, eps, offset), r


def layer_norm(x, weight, bias, eps: float = 1e-6):
    if _use_cuda(x):
        return _cu().layer_norm(x, weight, bias, eps)
    return ref.layer_norm(x, weight, bias, eps)


def rms_norm_gated(x, z, weight, eps: float = 1e-6):
    if _use_cuda(x):
        return _cu().rms_norm_gated(x, z, weight, eps)
    return ref.rms_norm_gated(x, z, weight, eps)


# --- GEMM --------------------------------------------------------------------
def _ref_linear(x, weight, bias=None):
    """The CPU linear; a weight tagged for FP8 training (``parallel/float8.py``) goes through the FP8 emulation."""
    if getattr(weight, "_vlmt_fp8", False):
        from . import float8

        float8.CALLS["linear"] += 1
        return float8.linear_ref(x, weight, bias)
    return ref.linear(x, weight, bias)


def linear(x, weight, bias=None):
    if _use_cuda(x):
        return _cu().linear(x, weight, bias)
    return _ref_linear(x, weight, bias)


def linear_gelu(x, weight, bias, approximate: str = "tanh"):
    """``gelu(x @ W.T + b)`` — bias and activation run in the GEMM epilogue on CUDA."""
    if _use_cuda(x):
        return _cu().linear_gelu(x, weight, bias, approximate)
    y = _ref_linear(x, weight, bias)
    return ref.gelu_tanh(y) if approximate == "tanh" else ref.gelu_erf(y)


def rms_norm_linear(x, norm_weight, weight, eps: float = 1e-6, offset: bool = False, residual=None):
    """``linear(rms_norm(x + residual), weight)``; returns ``y`` or ``(y, x + residual)``.  On CUDA the normalised
    activation is not kept for backward (it is recomputed), which removes one ``[T, H]`` tensor per use."""
    if _use_cuda(x):
        return _cu().rms_norm_linear(x, norm_weight, weight, eps, offset, residual)
    if residual is None:
        return _ref_linear(ref.rms_norm(x, norm_weight, eps, offset), weight)
    r = x + residual
    return _ref_linear(ref.rms_norm(r, norm_weight, eps, offset), weight), r


def layer_norm_linear(x, ln_weight, ln_bias, weight, bias=None, eps: float = 1e-6):
    """``linear(layer_norm(x), weight, bias)``; on CUDA the normalised activation is recomputed in backward."""
    if _use_cuda(x):
        return _cu().layer_norm_linear(x, ln_weight, ln_bias, weight, bias, eps)
    return _ref_linear(ref.layer_norm(x, ln_weight, ln_bias, eps), weight, bias)


def gelu_linear(pre, weight, bias=None, approximate: str = "tanh"):
    """``linear(gelu(pre), weight, bias)``; on CUDA only ``pre`` is kept for backward."""
    if _use_cuda(pre):
        return _cu().gelu_linear(pre, weight, bias, approximate)
    act = ref.gelu_tanh(pre) if approximate == "tanh" else ref.gelu_erf(pre)
    return _ref_linear(act, weight, bias)


def swiglu_linear(gate_up, weight):
    """``linear(silu(gate) * up, weight)`` for a fused ``[T, 2I]`` input; on CUDA only ``gate_up`` is kept for backward."""
    if _use_cuda(gate_up):
        return _cu().swiglu_linear(gate_up, weight)
    g, u = gate_up.chunk(2, dim=-1)
    return _ref_linear(ref.swiglu(g, u), weight)


# --- activations -------------------------------------------------------------
def swiglu(gate_up):
    """``silu(gate) * up`` for a fused ``[..., 2I]`` tensor laid out ``[gate | up]``."""
    if _use_cuda(gate_up):
        return _cu().swiglu(gate_up)
    g, u = gate_up.chunk(2, dim=-1)
    return ref.swiglu(g, u)


def sigmoid_mul(x, gate):
    """``x * sigmoid(gate)`` (attention output gate of Qwen3.5)."""
    if _use_cuda(x):
        return _cu().sigmoid_mul(x, gate)
    return (x.float() * torch.sigmoid(gate.float())).to(x.dtype)


# --- rotary / qkv prep --------------------------------------------------------
def qkv_norm_rope(qkv, n_q: int, n_kv: int, head_dim: int, q_weight, k_weight, cos, sin,
                  eps: float = 1e-6, offset: bool = False, gated: bool = False):
    """Split a fused projection ``[T, (n_q*(2 if gated else 1) + 2*n_kv) * D]``
    into q, k, v (and the per-head output gate), apply per-head RMSNorm to q and
    k and rotary embedding to their first ``cos.shape[-1]`` channels.

    Returns ``(q [T,n_q,D], k [T,n_kv,D], v [T,n_kv,D], gate [T,n_q*D] | None)``.
    Replaces a chain of view/transpose/contiguous/elementwise ops
    (reference: models/qwen3_vl/model.py:256-269, models/qwen3_5/model.py:111-131).
    """
    if _use_cuda(qkv):
        return _cu().qkv_norm_rope(qkv, n_q, n_kv, head_dim, q_weight, k_weight, cos, sin, eps, offset, gated)
    T = qkv.shape[0]
    D = head_dim
    qw = n_q * D * (2 if gated else 1)
    q, k, v = qkv.split([qw, n_kv * D, n_kv * D], dim=-1)
    gate = None
    if gated:
        q, gate = q.view(T, n_q, 2 * D).chunk(2, dim=-1)
        gate = gate.reshape(T, n_q * D)
    q = q.reshape(T, n_q, D)
    k = k.reshape(T, n_kv, D)
    v = v.reshape(T, n_kv, D)
    if q_weight is not None:
        q, k = ref.rms_norm(q, q_weight, eps, offset), ref.rms_norm(k, k_weight, eps, offset)
    q, k = ref.apply_rope(q, cos, sin), ref.apply_rope(k, cos, sin)
    return q, k, v, gate


def rope_vision(q, k, cos, sin, pad_to=None):
    """fp32 rotate-half rotary on ViT q,k ``[S, H, D]`` with ``cos/sin [S, D]``
    (reference: models/qwen3_vl/model.py:385-394).  ``pad_to`` appends zero channels up to that width."""
    if _use_cuda(q):
        return _cu().rope_vision(q, k, cos, sin, pad_to)
    q, k = ref.apply_rope(q, cos, sin), ref.apply_rope(k, cos, sin)
    if pad_to and pad_to > q.shape[-1]:
        pad = (0, pad_to - q.shape[-1])
        q, k = torch.nn.functional.pad(q, pad), torch.nn.functional.pad(k, pad)
    return q, k


# --- attention ---------------------------------------------------------------
def attention_varlen(q, k, v, cu_seqlens, max_seqlen: int, causal: bool = True, scale: float | None = None):
    if _use_cuda(q):
        return _cu().attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale)
    return ref.attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale)


def dsa_attention(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk: int, scale: float | None = None, cu_host=None):
    """``cu_host``: the document boundaries as a host sequence, if the caller has them (no device read then)."""
    if _use_cuda(q):
        return _cu().dsa_attention(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk, scale, cu_host)
    return ref.dsa_attention(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk, scale)


# --- loss --------------------------------------------------------------------
def linear_cross_entropy(hidden, weight, targets, chunk: int = 1024, ignore_index: int = -100):
    if _use_cuda(hidden):
        return _cu().linear_cross_entropy(hidden, weight, targets, chunk, ignore_index)
    return ref.linear_cross_entropy(hidden, weight, targets, chunk, ignore_index)


# --- gated delta net ---------------------------------------------------------
def causal_conv1d_silu(x, weight, seq_idx):
    if _use_cuda(x):
        return _cu().causal_conv1d_silu(x, weight, seq_idx)
    return ref.causal_conv1d_silu(x, weight, seq_idx)


def gdn_gates(a, b, A_log, dt_bias):
    """``g = -exp(A_log) * softplus(a + dt_bias)`` (fp32) and ``beta = sigmoid(b)``
    (reference: models/qwen3_5/model.py:226-227)."""
    if _use_cuda(a):
        return _cu().gdn_gates(a, b, A_log, dt_bias)
    g = -A_log.float().exp() * torch.nn.functional.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float()).to(b.dtype)


def gated_delta_rule(q, k, v, g, beta, cu_seqlens, scale: float | None = None, chunk: int = 64, cu_host=None):
    """``cu_host``: the same boundaries as a host sequence (saves a device sync when given)."""
    if _use_cuda(q):
        return _cu().gated_delta_rule(q, k, v, g, beta, cu_seqlens, scale, chunk, cu_host)
    return ref.gated_delta_rule(q, k, v, g, beta, cu_seqlens, scale, chunk)


# --- MoE ---------------------------------------------------------------------
def moe_router(logits, top_k: int, renorm: bool = True):
    if _use_cuda(logits):
        return _cu().moe_router(logits, top_k, renorm)
    return ref.moe_router(logits, top_k, renorm)


def moe_experts(x, gate_up, down, weights, experts):
    if _use_cuda(x):
        return _cu().moe_experts(x, gate_up, down, weights, experts)
    return ref.moe_experts(x, gate_up, down, weights, experts)


# --- vision glue -------------------------------------------------------------
def scatter_rows(x, index, src):
    if _use_cuda(x):
        return _cu().scatter_rows(x, index, src)
    return ref.scatter_rows(x, index, src)


def add_rows(x, index, src):
    if _use_cuda(x):
        return _cu().add_rows(x, index, src)
    return ref.add_rows(x, index, src)


def embedding(ids, weight):
    return torch.nn.functional.embedding(ids, weight)
