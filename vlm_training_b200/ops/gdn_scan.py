"""Gated delta rule over a packed row with the chunk-to-chunk recurrence as one scan kernel.

Same maths as :func:`vlm_training_b200.ops.reference.gated_delta_rule` (WY / UT chunk form, chunk 64, state reset
at every document boundary; reference: models/qwen3_5/model.py:180-186 calls fla's ``chunk_gated_delta_rule``),
split by what can run in parallel:

* inside a chunk (decay matrices, the 64x64 triangular solve, ``w``, ``u``, the local attention matrix ``P``):
  batched over all chunks of all documents and heads: on a GPU the kernels of ``csrc/gdn_chunk_sm100.cu`` (one CTA per chunk
  and head; :class:`_ChunkedNative`), else plain tensor operations with autograd;
* between chunks: ``vnew_c = u_c - w_c S_c`` and ``S_{c+1} = S_c exp(g_last) + kdec_c^T vnew_c``.  This is the only
  sequential part and runs as :func:`scan` — on a GPU one tcgen05 kernel launch for all documents and heads
  (``csrc/gdn_scan_sm100.cu``), which also writes the state entering every chunk;
* the outputs ``o_c = (q e^{gc}) S_c + P vnew_c`` then need no recurrence and are batched GEMMs again.

The backward of the scan is the same scan run over the chunks in reverse (the adjoint state ``G`` takes the place of
``S``), followed by batched products for ``dw``, ``dkdec`` and the decay gradient; see :class:`_Scan`.

The scan, in the form both directions share (state ``Z [Dv, Dk]`` per document and head, zero at the first step)::

    states[c] = Z                                   # the state entering step c
    Y[c]      = E[c] + s1 * (X1[c] Z^T)             # [C, Dv]
    Z         = ext[c] + decay[c] * Z + s2 * Y[c]^T X2[c]

forward: ``X1 = w, X2 = kdec, E = u, s1 = -1, s2 = +1, ext = 0`` gives ``Y = vnew`` and ``states = S^T``;
backward: ``X1 = kdec, X2 = w, E = dvnew, s1 = +1, s2 = -1, ext = dS`` over the chunks in reverse gives the total
``dvnew`` and the adjoint states.
"""
from __future__ import annotations

import numpy as np
import torch

from .reference import l2norm

CHUNK = 64


def doc_chunk_ranges(cu_host, chunk: int = CHUNK):
    """Documents' chunks laid out one document after the other.  Returns ``(dst, n_chunks, first, count)``:
    ``dst[t]`` is token ``t``'s row in the padded ``[n_chunks * chunk]`` layout, ``first`` / ``count`` the chunk range
    of every non-empty document (numpy int32)."""
    cu = np.asarray(cu_host, dtype=np.int64)
    lens = np.diff(cu)
    keep = lens > 0
    n_per = (lens + chunk - 1) // chunk
    first_all = np.concatenate(([0], np.cumsum(n_per)))[:-1]
    T = int(cu[-1])
    tok = np.arange(T)
    doc = np.searchsorted(cu[1:], tok, side="right")
    dst = first_all[doc] * chunk + (tok - cu[doc])
    return dst, int(n_per.sum()), first_all[keep].astype(np.int32), n_per[keep].astype(np.int32)


def scan_torch(x1, x2, e, decay, ext, first, count, reverse: bool, head_major: bool = False):
    """The scan as a loop of tensor operations (CPU, and the statement the kernel is tested against).
    ``x1, x2 [N,H,C,Dk]``, ``e [N,H,C,Dv]``, ``decay [N,H]``, ``ext [N,H,Dv,Dk]`` or ``None``
    (``head_major``: the first two dimensions exchanged, in and out).
    Returns ``(Y [N,H,C,Dv], states [N,H,Dv,Dk])`` in float32."""
    if head_major:
        y, st = scan_torch(x1.transpose(0, 1), x2.transpose(0, 1), e.transpose(0, 1), decay.transpose(0, 1),
                           ext.transpose(0, 1) if ext is not None else None, first, count, reverse)
        return y.transpose(0, 1).contiguous(), st.transpose(0, 1).contiguous()
    N, H, C, Dk = x1.shape
    Dv = e.shape[-1]
    s1, s2 = (1.0, -1.0) if reverse else (-1.0, 1.0)
    y = torch.empty(N, H, C, Dv, dtype=torch.float32, device=x1.device)
    states = torch.empty(N, H, Dv, Dk, dtype=torch.float32, device=x1.device)
    x1f, x2f, ef = x1.float(), x2.float(), e.float()
    for f, n in zip(first.tolist(), count.tolist()):
        z = torch.zeros(H, Dv, Dk, dtype=torch.float32, device=x1.device)
        order = range(f + n - 1, f - 1, -1) if reverse else range(f, f + n)
        for c in order:
            states[c] = z
            yc = ef[c] + s1 * (x1f[c] @ z.transpose(-1, -2))
            y[c] = yc
            z = decay[c].float().view(H, 1, 1) * z + s2 * (yc.transpose(-1, -2) @ x2f[c])
            if ext is not None:
                z = z + ext[c].float()
    return y, states


def _scan_impl(x1, x2, e, decay, ext, ranges, reverse):
    if x1.is_cuda:
        from . import cuda as cu

        return cu.gdn_scan(x1, x2, e, decay, ext, ranges, reverse, head_major=True)
    first, count = ranges[0], ranges[1]
    return scan_torch(x1, x2, e, decay, ext, first, count, reverse, head_major=True)


class _Scan(torch.autograd.Function):
    """``(w, u, kdec, decay) -> (S_all^T [H,N,Dv,Dk], vnew [H,N,C,Dv])``; all tensors head-major ``[H, N, ...]``.

    Backward, with ``G_c`` the gradient with respect to the state entering chunk ``c + 1`` accumulated over everything
    that follows it: ``dvnew_c = dvnew_ext_c + kdec_c G_c``, ``G_{c-1} = dS_ext_c + decay_c G_c - w_c^T dvnew_c`` (the
    reverse scan), then ``du = dvnew``, ``dw_c = -dvnew_c S_c^T``, ``dkdec_c = vnew_c G_c^T``,
    ``ddecay_c = <S_c, G_c>``."""

    @staticmethod
    def forward(ctx, w, u, kdec, decay, ranges):
        vnew, states = _scan_impl(w, kdec, u, decay, None, ranges, False)
        ctx.ranges = ranges
        ctx.save_for_backward(w, kdec, decay, vnew, states)
        ctx.in_dtypes = (w.dtype, u.dtype, kdec.dtype, decay.dtype)
        return states, vnew

    @staticmethod
    def backward(ctx, d_states, d_vnew):
        w, kdec, decay, vnew, states = ctx.saved_tensors
        if d_vnew is None:
            d_vnew = torch.zeros_like(vnew)
        if d_vnew.dtype != vnew.dtype:
            d_vnew = d_vnew.to(vnew.dtype)
        dv_tot, adj = _scan_impl(kdec, w, d_vnew.contiguous(), decay, d_states.contiguous() if d_states is not None else None,
                                 ctx.ranges, True)
        wt, ut, kt, dt = ctx.in_dtypes
        dw = -(dv_tot @ states.to(dv_tot.dtype))                     # [C,Dv] @ [Dv,Dk]
        dkdec = vnew.to(adj.dtype) @ adj
        ddecay = (states.float() * adj.float()).sum((-1, -2))
        return dw.to(wt), dv_tot.to(ut), dkdec.to(kt), ddecay.to(dt), None


def chunk_table(cu_host, chunk: int = CHUNK):
    """Per chunk slot (the order :func:`doc_chunk_ranges` lays them out in): first token and number of rows, ``int32 [N, 2]``."""
    cu = np.asarray(cu_host, dtype=np.int64)
    lens = np.diff(cu)
    n_per = (lens + chunk - 1) // chunk
    doc = np.repeat(np.arange(len(lens)), n_per)
    first_all = np.concatenate(([0], np.cumsum(n_per)))[:-1]
    idx = np.arange(int(n_per.sum())) - np.repeat(first_all, n_per)
    tok0 = cu[doc] + idx * chunk
    rows = np.minimum(chunk, cu[doc + 1] - tok0)
    return np.stack((tok0, rows), 1).astype(np.int32)


_TABLES: dict = {}
NATIVE_CALLS = {"forward": 0, "backward": 0}   # how often the all-kernel path ran (tests assert on it)


def _device_tables(cu_host, device):
    """Chunk table and document ranges on the device, kept for the last few packed rows (every linear-attention layer
    of a step, and its recomputation, asks for the same one)."""
    key = (tuple(int(x) for x in cu_host), str(device))
    hit = _TABLES.get(key)
    if hit is None:
        _dst, n_slots, first, count = doc_chunk_ranges(cu_host)
        chunks = torch.from_numpy(chunk_table(cu_host)).to(device, non_blocking=True)
        ranges = (first, count, torch.from_numpy(np.stack((first, count), 1).copy()).to(device, non_blocking=True))
        hit = (chunks, ranges, n_slots)
        if len(_TABLES) >= 8:
            _TABLES.pop(next(iter(_TABLES)))
        _TABLES[key] = hit
    return hit


class _ChunkedNative(torch.autograd.Function):
    """The whole rule on a GPU: prepare -> scan -> output, each one kernel launch (``csrc/gdn_chunk_sm100.cu``,
    ``csrc/gdn_scan_sm100.cu``), and the same three stages in reverse for the gradients.  Saved for backward: the scan
    operands and results, ``P``, the triangular inverse and the cumulative decays (all bf16 tile stacks)."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, chunks, ranges, scale, covered):
        from . import cuda as cu

        NATIVE_CALLS["forward"] += 1
        gf, bf = g.float().contiguous(), beta.float().contiguous()
        w, u, kdec, qg, P, Tm, gc, decay = cu._C.gdn_prepare_fwd(q, k, v, gf, bf, chunks, scale, 1e-6)
        vnew, states = cu.gdn_scan(w, kdec, u, decay, None, ranges, False, head_major=True)
        o = cu._C.gdn_output_fwd(qg, P, states, vnew, chunks, q.shape[0], covered)
        cu._tick(2)
        ctx.save_for_backward(q, k, v, bf, gc, decay, w, kdec, qg, P, Tm, vnew, states, chunks)
        ctx.ranges, ctx.scale, ctx.covered = ranges, scale, covered
        ctx.dtypes = (g.dtype, beta.dtype)
        return o

    @staticmethod
    def backward(ctx, do):
        from . import cuda as cu

        NATIVE_CALLS["backward"] += 1
        q, k, v, bf, gc, decay, w, kdec, qg, P, Tm, vnew, states, chunks = ctx.saved_tensors
        dqg, dP, dvn, dS = cu._C.gdn_output_bwd(do.contiguous(), qg, P, states, vnew, chunks)
        du, adj = cu.gdn_scan(kdec, w, dvn, decay, dS, ctx.ranges, True, head_major=True)
        dq, dk, dv, dg, dbeta = cu._C.gdn_prepare_bwd(q, k, v, bf, gc, chunks, ctx.scale, 1e-6, states, adj, vnew, du, dqg, dP, P, Tm,
                                                      ctx.covered)
        cu._tick(2)
        return dq, dk, dv, dg.to(ctx.dtypes[0]), dbeta.to(ctx.dtypes[1]), None, None, None, None


def native_usable(q, k, v, chunk) -> bool:
    import os

    def tokens_ok(t):
        return t.dim() == 3 and t.stride(2) == 1 and t.stride(1) == 128 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0

    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and chunk == CHUNK
            and q.shape[-1] == 128 and v.shape[-1] == 128 and q.shape == k.shape == v.shape and all(tokens_ok(t) for t in (q, k, v))
            and os.environ.get("VLMT_GDN_CHUNK", "1") != "0")


def gated_delta_rule_scan(q, k, v, g, beta, cu_host, scale=None, chunk: int = CHUNK, work_dtype=None):
    """``q, k [T,H,Dk]``, ``v [T,H,Dv]``, ``g, beta [T,H]``; ``cu_host`` the document boundaries as a host sequence.
    ``work_dtype``: dtype of the scan's operands and states (bf16 on a GPU, float32 on CPU)."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    dev = q.device
    if work_dtype is None:
        work_dtype = torch.bfloat16 if q.is_cuda else torch.float32
    scale = scale if scale is not None else Dk ** -0.5
    if work_dtype is torch.bfloat16 and native_usable(q, k, v, chunk):
        chunks, ranges, _n = _device_tables(cu_host, dev)
        covered = int(np.asarray(cu_host)[-1]) == T and int(np.asarray(cu_host)[0]) == 0   # every token belongs to a chunk
        return _ChunkedNative.apply(q, k, v, g, beta, chunks, ranges, float(scale), covered)
    dst_np, n_slots, first, count = doc_chunk_ranges(cu_host, chunk)
    Tc = int(np.asarray(cu_host)[-1])
    dst = torch.from_numpy(dst_np).to(dev, non_blocking=True)
    ranges = (first, count, torch.from_numpy(np.stack((first, count), 1).copy()).to(dev, non_blocking=True))

    # Head-major padded layout [H, n_slots, chunk, ...]: one index_copy per tensor writes it contiguously, so the batched
    # products below never re-copy a transposed view.  Padding rows are zero and have no effect.
    def pad(x):  # [T, H, ...] -> [H, n_slots, chunk, ...]
        xt = x[:Tc].transpose(0, 1)
        out = xt.new_zeros((H, n_slots * chunk) + tuple(x.shape[2:]))
        out.index_copy_(1, dst, xt)
        return out.view(H, n_slots, chunk, *x.shape[2:])

    qf = l2norm(pad(q)) * scale
    kf = l2norm(pad(k))
    vf = pad(v).float()
    gf = pad(g.float())        # [H, N, C]
    bf = pad(beta.float())
    gc = gf.cumsum(-1)
    kb = kf * bf.unsqueeze(-1)
    vb = vf * bf.unsqueeze(-1)
    dec = gc.unsqueeze(-1) - gc.unsqueeze(-2)  # [N, H, C, C]: gc_i - gc_j
    incl = torch.ones(chunk, chunk, dtype=torch.bool, device=dev).tril(0)
    decay_incl = dec.masked_fill(~incl, float("-inf")).exp()      # exp(gc_i - gc_j) for j <= i, else 0
    A = (kb @ kf.transpose(-1, -2)) * decay_incl.tril(-1)
    eye = torch.eye(chunk, device=dev, dtype=torch.float32)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    w = Tm @ (kb * gc.exp().unsqueeze(-1))
    u = Tm @ vb
    P = (qf @ kf.transpose(-1, -2)) * decay_incl
    qg = qf * gc.exp().unsqueeze(-1)
    last = gc[..., -1]
    kdec = kf * (last.unsqueeze(-1) - gc).exp().unsqueeze(-1)
    states, vnew = _Scan.apply(w.to(work_dtype).contiguous(), u.to(work_dtype).contiguous(),
                               kdec.to(work_dtype).contiguous(), last.exp().contiguous(), ranges)
    o = qg.to(work_dtype) @ states.transpose(-1, -2) + P.to(work_dtype) @ vnew      # [H, N, C, Dv]
    out = o.reshape(H, n_slots * chunk, Dv).index_select(1, dst).transpose(0, 1)     # [Tc, H, Dv]
    if Tc < T:
        out = torch.cat((out, out.new_zeros(T - Tc, H, Dv)), 0)
    return out.to(v.dtype)
