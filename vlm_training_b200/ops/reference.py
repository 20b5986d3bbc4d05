"""Plain-PyTorch statements of every hot op.

These are the oracles the CUDA kernels are tested against (run in fp32) and the
implementation used when the tensors live on the CPU (gloo runs, unit tests).
Everything here is differentiable through autograd; nothing here is tuned.

Shapes use ``T`` = tokens of one packed row, ``H`` = heads, ``D`` = head dim.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- norms
def rms_norm(x, weight, eps: float, offset: bool = False):
    """``x * rsqrt(mean(x^2) + eps) * w`` in fp32, cast back to ``x.dtype``;
    ``offset`` selects the Qwen3.5 form ``(1 + w)``
    (reference: models/qwen3_5/model.py:58-72, models/qwen3/model.py:73-84)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float()
    y = y * (1.0 + w) if offset else y * w
    return y.to(x.dtype)


def layer_norm(x, weight, bias, eps: float):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


def rms_norm_gated(x, z, weight, eps: float):
    """``rms_norm(x) * w * silu(z)`` per row of the last dim
    (reference: models/qwen3_5/model.py:32-56)."""
    xf, zf = x.float(), z.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return (y * zf * torch.sigmoid(zf)).to(x.dtype)


# --------------------------------------------------------------------------- activations
def swiglu(gate, up):
    g = gate.float()
    return (g * torch.sigmoid(g) * up.float()).to(gate.dtype)


def gelu_tanh(x):
    return F.gelu(x, approximate="tanh")


def gelu_erf(x):
    return F.gelu(x)


def linear(x, weight, bias=None):
    return F.linear(x, weight, bias)


# --------------------------------------------------------------------------- rotary
def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x, cos, sin):
    """Rotate the first ``cos.shape[-1]`` channels of ``x [T, H, D]`` with
    ``cos/sin [T, R]``; channels beyond R pass through (partial rotary,
    reference: models/qwen3_5/utils.py:88-110)."""
    r = cos.shape[-1]
    c = cos.unsqueeze(1).float()
    s = sin.unsqueeze(1).float()
    xr = x[..., :r].float()
    out = xr * c + rotate_half(xr) * s
    if r == x.shape[-1]:
        return out.to(x.dtype)
    return torch.cat((out.to(x.dtype), x[..., r:]), dim=-1)


def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps: float, offset: bool = False):
    """Per-head RMSNorm on q and k followed by rotary embedding.
    q ``[T, Hq, D]``, k ``[T, Hkv, D]``, cos/sin ``[T, R]``."""
    q = rms_norm(q, q_weight, eps, offset)
    k = rms_norm(k, k_weight, eps, offset)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin)


def mrope_cos_sin(position_ids, inv_freq, mrope_section, dtype=torch.float32):
    """Interleaved multi-axis rotary table.

    ``position_ids [3, T]`` (temporal, height, width), ``inv_freq [R/2]``.
    Frequency index ``j`` takes the height position when ``j % 3 == 1`` and
    ``j < 3*section[1]``, the width position when ``j % 3 == 2`` and
    ``j < 3*section[2]``, else the temporal one
    (reference: models/qwen3_vl/model.py:196-222).  Returns cos, sin ``[T, R]``.
    """
    freqs = position_ids.float().unsqueeze(-1) * inv_freq.float()  # [3, T, R/2]
    n = inv_freq.shape[0]
    j = torch.arange(n, device=freqs.device)
    use_h = (j % 3 == 1) & (j < 3 * mrope_section[1])
    use_w = (j % 3 == 2) & (j < 3 * mrope_section[2])
    f = torch.where(use_h, freqs[1], torch.where(use_w, freqs[2], freqs[0]))
    emb = torch.cat((f, f), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


# --------------------------------------------------------------------------- attention
def attention_varlen(q, k, v, cu_seqlens, max_seqlen: int | None = None, causal: bool = True,
                     scale: float | None = None, topk_idx=None):
    """Block-diagonal (per document) softmax attention over a packed row.

    q ``[T, Hq, D]``, k/v ``[T, Hkv, D]`` with ``Hq % Hkv == 0``; documents are
    ``[cu[i], cu[i+1])``.  fp32 math, output in ``q.dtype``
    (reference behaviour: torch varlen_attn, models/qwen3_vl/model.py:25-46).
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cu = [int(c) for c in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]
    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        qs = q[s:e].float().transpose(0, 1)  # [Hq, L, D]
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        att = (qs @ ks.transpose(-1, -2)) * scale
        L = e - s
        if causal:
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            att = att.masked_fill(~mask, float("-inf"))
        p = att.softmax(-1)
        outs.append((p @ vs).transpose(0, 1))
    if cu[-1] < T:  # rows past the last boundary attend to nothing
        outs.append(torch.zeros(T - cu[-1], Hq, v.shape[-1], device=q.device))
    return torch.cat(outs, 0).to(q.dtype)


def dsa_attention(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk: int, scale: float | None = None):
    """Sparse attention: each query keeps only the ``topk`` causal keys of its
    document ranked by an indexer score, then runs softmax attention over them.

    Indexer score for query t and key s: ``sum_h idx_w[t,h] * relu(idx_q[t,h]·idx_k[s])``
    with ``idx_q [T, Hi, Di]``, ``idx_k [T, Di]``, ``idx_w [T, Hi]``.
    The oracle is dense attention under the same top-k mask.
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cu = [int(c) for c in cu_seqlens.tolist()]
    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        L = e - s
        sc = torch.einsum("thd,sd->ths", idx_q[s:e].float(), idx_k[s:e].float()).relu()
        sc = (sc * idx_w[s:e].float().unsqueeze(-1)).sum(1)  # [L, L]
        causal = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~causal, float("-inf"))
        keep = causal
        if L > topk:
            kth = sc.topk(topk, dim=-1).indices
            sel = torch.zeros(L, L, dtype=torch.bool, device=q.device).scatter_(1, kth, True)
            keep = causal & sel
        qs = q[s:e].float().transpose(0, 1)
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        att = (qs @ ks.transpose(-1, -2)) * scale
        att = att.masked_fill(~keep, float("-inf"))
        outs.append((att.softmax(-1) @ vs).transpose(0, 1))
    if cu[-1] < T:
        outs.append(torch.zeros(T - cu[-1], Hq, v.shape[-1], device=q.device))
    return torch.cat(outs, 0).to(q.dtype)


# --------------------------------------------------------------------------- loss
def linear_cross_entropy(hidden, weight, targets, chunk: int = 1024, ignore_index: int = -100):
    """Sum of token cross-entropies of ``hidden @ weight.T`` against ``targets``
    without materialising more than ``chunk`` rows of logits at a time.

    hidden ``[T, H]``, weight ``[V, H]``, targets ``[T]`` (already shifted).
    Returns ``(loss_sum fp32 scalar, n_valid int64 scalar)``; the mean loss of
    the unchunked reference (reference: models/qwen3_vl/model.py:834-840) is
    ``loss_sum / n_valid``.
    """
    T = hidden.shape[0]
    total = hidden.new_zeros((), dtype=torch.float32)
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        logits = F.linear(hidden[s:e], weight).float()
        total = total + F.cross_entropy(logits, targets[s:e], ignore_index=ignore_index, reduction="sum")
    n_valid = (targets != ignore_index).sum()
    return total, n_valid


# --------------------------------------------------------------------------- gated delta net
def seq_idx_from_cu(cu_seqlens, T: int, device=None):
    """Document index of every token: ``#{boundaries in cu[1:-1] <= t}``
    (reference: models/qwen3_5/model.py:198-200)."""
    device = device if device is not None else cu_seqlens.device
    pos = torch.arange(T, device=device)
    return torch.bucketize(pos, cu_seqlens[1:-1].to(device), right=True).to(torch.int32)


def causal_conv1d_silu(x, weight, seq_idx):
    """Depthwise causal convolution over a packed row followed by SiLU.

    x ``[T, C]``, weight ``[C, K]``, seq_idx ``[T]``:
    ``y[t,c] = silu(sum_j w[c,j] * x[t-(K-1)+j, c])`` where taps that fall
    before the start of t's document contribute 0
    (reference: models/qwen3_5/model.py:174-176,203-208)."""
    T, C = x.shape
    K = weight.shape[1]
    xf = x.float()
    acc = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    for j in range(K):
        shift = K - 1 - j
        if shift == 0:
            acc = acc + xf * weight[:, j].float()
            continue
        xs = torch.cat((torch.zeros(shift, C, device=x.device), xf[:-shift]), 0) if shift < T else torch.zeros_like(xf)
        same = torch.cat((torch.zeros(shift, dtype=torch.bool, device=x.device),
                          seq_idx[shift:] == seq_idx[:-shift]), 0) if shift < T else torch.zeros(T, dtype=torch.bool, device=x.device)
        acc = acc + torch.where(same.unsqueeze(-1), xs, torch.zeros_like(xs)) * weight[:, j].float()
    return (acc * torch.sigmoid(acc)).to(x.dtype)


def l2norm(x, eps: float = 1e-6):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)


def gated_delta_rule_recurrent(q, k, v, g, beta, cu_seqlens, scale: float | None = None, l2norm_qk: bool = True):
    """Token-by-token gated delta rule; the definitional oracle.

    q,k ``[T, H, Dk]``, v ``[T, H, Dv]``, g (log decay ≤ 0) and beta ``[T, H]``.
    Per document and head, with state ``S [Dk, Dv] = 0`` at the start:
    ``S ← S·exp(g_t)``; ``u = β_t (v_t − Sᵀ k_t)``; ``S ← S + k_t uᵀ``;
    ``o_t = Sᵀ (q_t·scale)`` (math spec: fla ops/gated_delta_rule/naive.py:13-64).
    """
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = scale if scale is not None else Dk ** -0.5
    qf = l2norm(q) if l2norm_qk else q.float()
    kf = l2norm(k) if l2norm_qk else k.float()
    vf, gf, bf = v.float(), g.float(), beta.float()
    qf = qf * scale
    cu = [int(c) for c in cu_seqlens.tolist()]
    out = torch.zeros(T, H, Dv, dtype=torch.float32, device=q.device)
    for s, e in zip(cu[:-1], cu[1:]):
        S = torch.zeros(H, Dk, Dv, dtype=torch.float32, device=q.device)
        for t in range(s, e):
            S = S * gf[t].exp().view(H, 1, 1)
            kv = torch.einsum("hk,hkv->hv", kf[t], S)
            u = bf[t].unsqueeze(-1) * (vf[t] - kv)
            S = S + torch.einsum("hk,hv->hkv", kf[t], u)
            out[t] = torch.einsum("hk,hkv->hv", qf[t], S)
    return out.to(v.dtype)


def _gdr_chunk_doc(q, k, v, g, beta, chunk: int):
    """Chunked (WY / UT transform) gated delta rule for ONE document.
    q,k [L,H,Dk] already normalised and scaled; returns [L,H,Dv] fp32."""
    L, H, Dk = q.shape
    Dv = v.shape[-1]
    pad = (-L) % chunk
    if pad:
        q = F.pad(q, (0, 0, 0, 0, 0, pad))
        k = F.pad(k, (0, 0, 0, 0, 0, pad))
        v = F.pad(v, (0, 0, 0, 0, 0, pad))
        g = F.pad(g, (0, 0, 0, pad))
        beta = F.pad(beta, (0, 0, 0, pad))
    n = (L + pad) // chunk
    # [H, n, C, *]
    q = q.permute(1, 0, 2).reshape(H, n, chunk, Dk)
    k = k.permute(1, 0, 2).reshape(H, n, chunk, Dk)
    v = v.permute(1, 0, 2).reshape(H, n, chunk, Dv)
    g = g.permute(1, 0).reshape(H, n, chunk)
    beta = beta.permute(1, 0).reshape(H, n, chunk)
    gc = g.cumsum(-1)  # inclusive cumulative log decay within the chunk
    kb = k * beta.unsqueeze(-1)
    vb = v * beta.unsqueeze(-1)
    decay = (gc.unsqueeze(-1) - gc.unsqueeze(-2))  # [.., i, j] = gc_i - gc_j
    strict = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril(-1)
    incl = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril(0)
    A = (kb @ k.transpose(-1, -2)) * decay.masked_fill(~strict, float("-inf")).exp()
    # (I + A)^-1 by forward substitution; A is strictly lower triangular
    eye = torch.eye(chunk, device=q.device, dtype=q.dtype)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    w = Tm @ (kb * gc.exp().unsqueeze(-1))
    u = Tm @ vb
    qk = (q @ k.transpose(-1, -2)) * decay.masked_fill(~incl, float("-inf")).exp()
    S = torch.zeros(H, Dk, Dv, dtype=q.dtype, device=q.device)
    outs = []
    for c in range(n):
        vnew = u[:, c] - w[:, c] @ S
        o = (q[:, c] * gc[:, c].exp().unsqueeze(-1)) @ S + qk[:, c] @ vnew
        outs.append(o)
        last = gc[:, c, -1]
        kdec = k[:, c] * (last.unsqueeze(-1) - gc[:, c]).exp().unsqueeze(-1)
        S = S * last.exp().view(H, 1, 1) + kdec.transpose(-1, -2) @ vnew
    o = torch.stack(outs, 1).reshape(H, n * chunk, Dv).permute(1, 0, 2)
    return o[:L]


def gated_delta_rule(q, k, v, g, beta, cu_seqlens, scale: float | None = None, chunk: int = 64,
                     l2norm_qk: bool = True):
    """Chunk-parallel form of :func:`gated_delta_rule_recurrent`; same maths,
    ``O(T·chunk)`` instead of a token loop.  State resets at every document
    boundary (reference: models/qwen3_5/model.py:180-186)."""
    T, H, Dk = q.shape
    scale = scale if scale is not None else Dk ** -0.5
    qf = (l2norm(q) if l2norm_qk else q.float()) * scale
    kf = l2norm(k) if l2norm_qk else k.float()
    vf, gf, bf = v.float(), g.float(), beta.float()
    cu = [int(c) for c in cu_seqlens.tolist()]
    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        outs.append(_gdr_chunk_doc(qf[s:e], kf[s:e], vf[s:e], gf[s:e], bf[s:e], chunk))
    if cu[-1] < T:
        outs.append(torch.zeros(T - cu[-1], H, v.shape[-1], device=q.device))
    return torch.cat(outs, 0).to(v.dtype)


# --------------------------------------------------------------------------- MoE
def moe_router(logits, top_k: int, renorm: bool = True):
    """softmax over experts → top-k → renormalise
    (HF Qwen3_5MoeTopKRouter, transformers qwen3_5_moe/modeling_qwen3_5_moe.py:754-770).
    Returns ``(weights [T,k] fp32, experts [T,k] int64)``."""
    p = logits.float().softmax(-1)
    w, idx = p.topk(top_k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


def moe_experts(x, gate_up, down, weights, experts):
    """Routed SwiGLU experts.  x ``[T,H]``, gate_up ``[E,2I,H]``, down ``[E,H,I]``,
    weights/experts ``[T,k]``.  Token t gets ``sum_j w[t,j] * expert_{e[t,j]}(x_t)``."""
    T, Hd = x.shape
    E = gate_up.shape[0]
    out = torch.zeros(T, Hd, dtype=torch.float32, device=x.device)
    for e in range(E):
        tok, slot = (experts == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        gu = F.linear(xe, gate_up[e])
        g, u = gu.chunk(2, dim=-1)
        h = swiglu(g, u)
        y = F.linear(h, down[e]).float() * weights[tok, slot].unsqueeze(-1).float()
        out.index_add_(0, tok, y)
    return out.to(x.dtype)


# --------------------------------------------------------------------------- vision glue
def scatter_rows(x, index, src):
    """Return a copy of ``x [T,H]`` whose rows ``index`` are replaced by ``src``
    (the index-list form of ``masked_scatter``, reference: models/qwen3_vl/model.py:774-777)."""
    return x.index_copy(0, index, src.to(x.dtype))


def add_rows(x, index, src):
    """``x[index] += src`` out of place (DeepStack injection,
    reference: models/qwen3_vl/model.py:329-333)."""
    return x.index_add(0, index, src.to(x.dtype))
