"""CUDA (sm_100a) implementations of the functional ops: autograd ``Function``s
over the compiled extension ``vlm_training_b200/ops/_C*.so``.

Importing this module loads the extension and raises if it is missing — there
is no fallback to PyTorch kernels for CUDA tensors.  GEMMs go through the
hand-written tcgen05 kernel (``gemm_sm100.cu``); set ``VLMT_GEMM=cublas`` to
route plain linears through ``torch.matmul`` instead (A/B comparison only).
"""
from __future__ import annotations

import importlib.util
import math
import os

import torch

from . import build as _build
from . import reference as ref


def _load_ext():
    path = _build.ext_path()
    if not os.path.exists(path):
        raise ImportError(
            f"compiled extension not found at {path}; run `python -m vlm_training_b200.ops.build` "
            "(or `__graft_entry__.build()`) first")
    spec = importlib.util.spec_from_file_location("vlm_training_b200.ops._C", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_C = _load_ext()
_GEMM_BACKEND = os.environ.get("VLMT_GEMM", "tcgen05")

# kernel-launch counter (bench.py reports how many of OUR kernels ran in the timed region)
LAUNCHES = {"count": 0}


def _tick(n: int = 1):
    LAUNCHES["count"] += n


def status_word() -> torch.Tensor:
    """The device status word of the current device (one int32): 0, or the code of the first bounded wait that ran out."""
    return _C.status()[:1]


def check_status(raise_on_error: bool = True) -> int:
    """Read (and clear) the device status word that bounded in-kernel waits write on timeout."""
    from . import status

    st = _C.status()
    if raise_on_error:
        return status.raise_if_set(st, "a kernel")
    code = int(st[0].item())
    if code != 0:
        st.zero_()
    return code


def debug_checks_enabled() -> bool:
    return os.environ.get("VLMT_DEBUG_CHECKS", "0") == "1"


def flag_if(bad: torch.Tensor, code: int):
    """Record ``code`` in the device status word where ``bad`` (a boolean device scalar) is true and no earlier code is set:
    no host read; the code surfaces with the step's metrics like a bounded wait that ran out."""
    st = status_word()
    st.copy_(torch.where(bad.reshape(1) & (st == 0), torch.full_like(st, code), st))


def validate_row_indices(cu_seqlens, n_tokens: int, image_rows=None, experts=None, n_experts: int = 0):
    """Debug aid (``VLMT_DEBUG_CHECKS=1``): the tensors from which kernels derive addresses.  ``cu_seqlens`` must start at
    0, be non-decreasing and end within the row (status 300); image rows must lie inside the row (301); expert ids inside
    ``[0, n_experts)`` (302).  Kernels index with these values unchecked, so a bad batch would otherwise be a stray access."""
    if cu_seqlens is not None:
        c = cu_seqlens.long()
        flag_if((c[0] != 0) | (c[1:] < c[:-1]).any() | (c[-1] > n_tokens), 300)
    if image_rows is not None and image_rows.numel():
        flag_if((image_rows < 0).any() | (image_rows >= n_tokens).any(), 301)
    if experts is not None and experts.numel():
        flag_if((experts < 0).any() | (experts >= n_experts).any(), 302)


# ------------------------------------------------------------------------------- GEMM
def _gemm(a, b, a_mn=False, b_mn=False, bias=None, epilogue=0, out=None, accumulate=False, out_dtype=torch.bfloat16):
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    pending = getattr(b, "_vlmt_wgather", None)
    if pending is not None:
        # a sharded weight whose gather was left to this GEMM (parallel/engine.py): its owners' parts arrive inside the kernel
        if (not a_mn and not b_mn and epilogue == 0 and not accumulate and out.dtype == torch.bfloat16 and a.dtype == torch.bfloat16
                and a.dim() == 2 and a.stride(1) == 1 and b.is_contiguous() and b.shape[0] > 128):
            pending.run(a, b, out, bias)
            _tick()
            return out
        pending.finish()
    if b.untyped_storage().size() == 0 or out.untyped_storage().size() == 0:
        # a sharded parameter (or its gradient bucket) whose storage is released: an error here, never a kernel on freed memory
        raise RuntimeError("GEMM operand without storage: a sharded parameter was used outside the forward / backward of its unit")
    _C.gemm(a, b, out, a_mn, b_mn, bias, epilogue, accumulate)
    _tick()
    return out


def _colsum(x2):
    """Column sums (a bias gradient) of a 2-D bf16 tensor in fp32; shapes the kernel does not take go through torch."""
    if x2.shape[1] % 8 == 0 and x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0 and x2.dtype == torch.bfloat16:
        _tick(2)
        return _C.colsum(x2)
    return x2.float().sum(0)


def _as_gemm_operand(t):
    """2-D, unit inner stride, 16-byte aligned row stride and base (TMA requirements)."""
    if t.stride(-1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def _tma_ok(*ts) -> bool:
    return all(t.shape[-1] % 8 == 0 and t.dtype == torch.bfloat16 for t in ts)


_WGRAD_IN_PLACE = os.environ.get("VLMT_WGRAD_IN_PLACE", "1") != "0"


def _grad_target(w):
    """The parameter whose ``.grad`` is a view of the optimizer engine's flat gradient buffer (the engine tags those),
    else ``None``.  Kept on the autograd context as a plain attribute: under activation checkpointing the tensors that
    come back from ``saved_tensors`` are detached copies without ``.grad``."""
    return w if (_WGRAD_IN_PLACE and getattr(w, "_vlmt_grad_in_place", False)) else None


def _wgrad(dy2, x2, param=None):
    """dW[N,K] = dY^T[N,M] . X[M,K].  For a tagged parameter the GEMM adds the product into ``param.grad`` from its
    epilogue (TMA reduce-add) and autograd gets ``None``: no separate accumulation pass over the gradient, no temporary.
    The engine's gradient-ready hook is called by hand because autograd has nothing to accumulate."""
    if param is not None:
        g = param.grad
        if (g is not None and g.dtype == torch.bfloat16 and g.dim() == 2 and g.shape == (dy2.shape[1], x2.shape[1])
                and g.stride(1) == 1 and g.stride(0) % 8 == 0 and g.data_ptr() % 16 == 0):
            _gemm(dy2, x2, a_mn=True, b_mn=True, out=g, accumulate=True)
            ready = getattr(param, "_vlmt_grad_ready", None)
            if ready is not None:
                ready(param)
            return None
    return _gemm(dy2, x2, a_mn=True, b_mn=True)


class _Linear(torch.autograd.Function):
    """y = x W^T (+ b).  fwd: (K,K) GEMM; dgrad: (K,MN); wgrad: (MN,MN) — no transposes materialised."""

    @staticmethod
    def forward(ctx, x, w, b, epilogue):
        x2 = _as_gemm_operand(x.reshape(-1, x.shape[-1]))
        wc = _as_gemm_operand(w)
        ctx.w_param = _grad_target(w)
        y = _gemm(x2, wc, bias=b, epilogue=epilogue)
        ctx.save_for_backward(x2, wc)
        ctx.has_bias = b is not None
        ctx.in_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _as_gemm_operand(dy.reshape(-1, dy.shape[-1]))
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _gemm(dy2, w, b_mn=True).view(ctx.in_shape)  # dX[M,K] = dY[M,N] . W[N,K]
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dy2, x2, ctx.w_param)  # dW[N,K] = dY^T[N,M] . X[M,K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _colsum(dy2).to(dy.dtype)
            _tick()
        return dx, dw, db, None


def _small_or_odd(x, w) -> bool:
    return (not _tma_ok(x, w)) or w.shape[0] < 16 or w.shape[0] % 8 != 0


def _fp8(weight) -> bool:
    """The weight was marked for FP8 training (``parallel/float8.py``): its linear goes through ``ops/float8.py``."""
    return getattr(weight, "_vlmt_fp8", False)


def linear(x, weight, bias=None):
    if _fp8(weight):
        from . import float8

        return float8.linear(x, weight, bias)
    if _GEMM_BACKEND == "cublas" or x.dtype != torch.bfloat16 or _small_or_odd(x, weight):
        return torch.nn.functional.linear(x, weight, bias)
    return _Linear.apply(x, weight, bias, 0)


def linear_gelu(x, weight, bias, approximate="tanh"):
    y = linear(x, weight, bias)
    return gelu(y, approximate)


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tanh_approx):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        ctx.tanh_approx = tanh_approx
        _tick()
        return _C.gelu_fwd(xc, tanh_approx)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        _tick()
        return _C.gelu_bwd(dy.contiguous(), x, ctx.tanh_approx), None


def gelu(x, approximate="tanh"):
    if x.dtype != torch.bfloat16 or x.numel() % 8:
        return torch.nn.functional.gelu(x, approximate="tanh" if approximate == "tanh" else "none")
    return _Gelu.apply(x, approximate == "tanh")


# ------------------------------------------------------------------------------- norms
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps, offset):
        xc = x.contiguous()
        if residual is None:
            y, rstd = _C.rmsnorm_fwd(xc, None, weight, eps, offset)
            ctx.save_for_backward(xc, weight, rstd)
            r = None
        else:
            y, rstd, r = _C.rmsnorm_fwd(xc, residual.contiguous(), weight, eps, offset)
            ctx.save_for_backward(r, weight, rstd)
        ctx.offset, ctx.has_res = offset, residual is not None
        _tick()
        if residual is None:
            return y
        return y, r

    @staticmethod
    def backward(ctx, dy, dr=None):
        x, w, rstd = ctx.saved_tensors
        dx, dw = _C.rmsnorm_bwd(dy.contiguous(), x, w, rstd, dr.contiguous() if dr is not None else None, ctx.offset)
        _tick(2)
        dw = dw.to(w.dtype)
        if ctx.has_res:
            return dx, dx, dw, None, None
        return dx, None, dw, None, None


def rms_norm(x, weight, eps=1e-6, offset=False):
    if x.dtype != torch.bfloat16 or x.shape[-1] % 8:
        return ref.rms_norm(x, weight, eps, offset)
    return _RMSNorm.apply(x, None, weight, eps, offset)


def add_rms_norm(x, residual, weight, eps=1e-6, offset=False):
    if x.dtype != torch.bfloat16 or x.shape[-1] % 8:
        r = x + residual
        return ref.rms_norm(r, weight, eps, offset), r
    return _RMSNorm.apply(x, residual, weight, eps, offset)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        xc = x.contiguous()
        y, mean, rstd = _C.layernorm_fwd(xc, weight, bias, eps)
        ctx.save_for_backward(xc, weight, mean, rstd)
        ctx.has_bias = bias is not None
        _tick()
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = _C.layernorm_bwd(dy.contiguous(), x, w, mean, rstd)
        _tick(3)
        return dx, dw.to(w.dtype), db.to(w.dtype) if ctx.has_bias else None, None


def layer_norm(x, weight, bias, eps=1e-6):
    if x.dtype != torch.bfloat16 or x.shape[-1] % 8:
        return ref.layer_norm(x, weight, bias, eps)
    return _LayerNorm.apply(x, weight, bias, eps)


class _RMSNormGated(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, z, weight, eps):
        xc, zc = x.contiguous(), z.contiguous()
        y, rstd = _C.rmsnorm_gated_fwd(xc, zc, weight, eps)
        ctx.save_for_backward(xc, zc, weight, rstd)
        _tick()
        return y

    @staticmethod
    def backward(ctx, dy):
        x, z, w, rstd = ctx.saved_tensors
        dx, dz, dw = _C.rmsnorm_gated_bwd(dy.contiguous(), x, z, w, rstd)
        _tick(2)
        return dx, dz, dw.to(w.dtype), None


def rms_norm_gated(x, z, weight, eps=1e-6):
    if x.dtype != torch.bfloat16:
        return ref.rms_norm_gated(x, z, weight, eps)
    return _RMSNormGated.apply(x, z, weight, eps)


# ------------------------------------------------------------------------------- activations
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        guc = gu.contiguous()
        ctx.save_for_backward(guc)
        _tick()
        return _C.swiglu_fwd(guc)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        _tick()
        return _C.swiglu_bwd(dout.contiguous(), gu)


def swiglu(gate_up):
    if gate_up.dtype != torch.bfloat16 or gate_up.shape[-1] % 16:
        g, u = gate_up.chunk(2, dim=-1)
        return ref.swiglu(g, u)
    return _SwiGLU.apply(gate_up)


class _SigmoidMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate):
        xc, gc = x.contiguous(), gate.contiguous()
        ctx.save_for_backward(xc, gc)
        _tick()
        return _C.sigmoid_mul_fwd(xc, gc)

    @staticmethod
    def backward(ctx, dout):
        x, g = ctx.saved_tensors
        _tick()
        dx, dg = _C.sigmoid_mul_bwd(dout.contiguous(), x, g)
        return dx, dg


def sigmoid_mul(x, gate):
    if x.dtype != torch.bfloat16 or x.shape != gate.shape or x.numel() % 8:
        return (x.float() * torch.sigmoid(gate.float())).to(x.dtype)
    return _SigmoidMul.apply(x, gate)


class _NormLinear(torch.autograd.Function):
    """``(x [+ residual]) → RMSNorm → linear`` that keeps only the un-normalised stream and ``rstd`` for backward;
    the normalised activation (the GEMM's A operand) is recomputed in backward by one cheap elementwise pass
    instead of being stored — 2 x T x H bytes less per use."""

    @staticmethod
    def forward(ctx, x, residual, norm_w, w, eps, offset):
        xc = x.contiguous()
        if residual is None:
            h, rstd = _C.rmsnorm_fwd(xc, None, norm_w, eps, offset)
            r = xc
        else:
            h, rstd, r = _C.rmsnorm_fwd(xc, residual.contiguous(), norm_w, eps, offset)
        wc = _as_gemm_operand(w)
        ctx.w_param = _grad_target(w)
        y = _gemm(h, wc)
        _tick()
        ctx.save_for_backward(r, norm_w, rstd, wc)
        ctx.cfg = (eps, offset, residual is not None)
        if residual is None:
            return y
        return y, r

    @staticmethod
    def backward(ctx, dy, dr=None):
        r, norm_w, rstd, w = ctx.saved_tensors
        eps, offset, has_res = ctx.cfg
        dy2 = _as_gemm_operand(dy)
        h = _C.rmsnorm_fwd(r, None, norm_w, eps, offset)[0]  # recompute the normalised activation
        dw = _wgrad(dy2, h, ctx.w_param)
        del h
        dh = _gemm(dy2, w, b_mn=True)
        dx, dnw = _C.rmsnorm_bwd(dh, r, norm_w, rstd, dr.contiguous() if dr is not None else None, offset)
        _tick(3)
        dnw = dnw.to(norm_w.dtype)
        if has_res:
            return dx, dx, dnw, dw, None, None
        return dx, None, dnw, dw, None, None


def rms_norm_linear(x, norm_weight, weight, eps=1e-6, offset=False, residual=None):
    """``linear(rms_norm(x + residual))``; returns ``y`` or ``(y, x + residual)``."""
    ok = x.dtype == torch.bfloat16 and _GEMM_BACKEND != "cublas" and not _small_or_odd(x, weight) and x.dim() == 2 and not _fp8(weight)
    if not ok:
        if residual is None:
            return linear(rms_norm(x, norm_weight, eps, offset), weight)
        h, r = add_rms_norm(x, residual, norm_weight, eps, offset)
        return linear(h, weight), r
    return _NormLinear.apply(x, residual, norm_weight, weight, eps, offset)


class _LNLinear(torch.autograd.Function):
    """``linear(layer_norm(x))`` keeping ``x`` and the row statistics; the normalised activation is recomputed in backward."""

    @staticmethod
    def forward(ctx, x, ln_w, ln_b, w, b, eps):
        xc = x.contiguous()
        h, mean, rstd = _C.layernorm_fwd(xc, ln_w, ln_b, eps)
        wc = _as_gemm_operand(w)
        ctx.w_param = _grad_target(w)
        y = _gemm(h, wc, bias=b)
        _tick()
        ctx.save_for_backward(xc, ln_w, ln_b, mean, rstd, wc)
        ctx.eps, ctx.has_bias = eps, b is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, ln_w, ln_b, mean, rstd, w = ctx.saved_tensors
        dy2 = _as_gemm_operand(dy)
        h = _C.layernorm_fwd(x, ln_w, ln_b, ctx.eps)[0]
        dw = _wgrad(dy2, h, ctx.w_param)
        del h
        dh = _gemm(dy2, w, b_mn=True)
        dx, dlw, dlb = _C.layernorm_bwd(dh, x, ln_w, mean, rstd)
        db = None
        if ctx.has_bias:
            db = _colsum(dy2).to(dy.dtype)
        _tick(4)
        return dx, dlw.to(ln_w.dtype), dlb.to(ln_w.dtype) if ln_b is not None else None, dw, db, None


def layer_norm_linear(x, ln_weight, ln_bias, weight, bias=None, eps=1e-6):
    ok = x.dtype == torch.bfloat16 and _GEMM_BACKEND != "cublas" and x.dim() == 2 and not _small_or_odd(x, weight) and not _fp8(weight)
    if not ok:
        return linear(layer_norm(x, ln_weight, ln_bias, eps), weight, bias)
    return _LNLinear.apply(x, ln_weight, ln_bias, weight, bias, eps)


class _GeluLinear(torch.autograd.Function):
    """``linear(gelu(pre))`` keeping only ``pre``; the activation is recomputed in backward."""

    @staticmethod
    def forward(ctx, pre, w, b, tanh_approx):
        pc = pre.contiguous()
        act = _C.gelu_fwd(pc, tanh_approx)
        wc = _as_gemm_operand(w)
        ctx.w_param = _grad_target(w)
        y = _gemm(act, wc, bias=b)
        _tick()
        ctx.save_for_backward(pc, wc)
        ctx.tanh_approx, ctx.has_bias = tanh_approx, b is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        pre, w = ctx.saved_tensors
        dy2 = _as_gemm_operand(dy)
        act = _C.gelu_fwd(pre, ctx.tanh_approx)
        dw = _wgrad(dy2, act, ctx.w_param)
        del act
        dact = _gemm(dy2, w, b_mn=True)
        dpre = _C.gelu_bwd(dact, pre, ctx.tanh_approx)
        db = None
        if ctx.has_bias:
            db = _colsum(dy2).to(dy.dtype)
        _tick(3)
        return dpre, dw, db, None


def gelu_linear(pre, weight, bias=None, approximate="tanh"):
    ok = (pre.dtype == torch.bfloat16 and _GEMM_BACKEND != "cublas" and pre.dim() == 2 and pre.numel() % 8 == 0
          and not _small_or_odd(pre, weight) and not _fp8(weight))
    if not ok:
        return linear(gelu(pre, approximate), weight, bias)
    return _GeluLinear.apply(pre, weight, bias, approximate == "tanh")


class _SwiGLULinear(torch.autograd.Function):
    """``linear(silu(gate) * up)`` that stores only ``gate_up``; the activation is recomputed in backward."""

    @staticmethod
    def forward(ctx, gate_up, w):
        guc = gate_up.contiguous()
        act = _C.swiglu_fwd(guc)
        wc = _as_gemm_operand(w)
        ctx.w_param = _grad_target(w)
        y = _gemm(act, wc)
        _tick()
        ctx.save_for_backward(guc, wc)
        return y

    @staticmethod
    def backward(ctx, dy):
        gu, w = ctx.saved_tensors
        dy2 = _as_gemm_operand(dy)
        act = _C.swiglu_fwd(gu)
        dw = _wgrad(dy2, act, ctx.w_param)
        del act
        dact = _gemm(dy2, w, b_mn=True)
        dgu = _C.swiglu_bwd(dact, gu)
        _tick(2)
        return dgu, dw


def swiglu_linear(gate_up, weight):
    ok = (gate_up.dtype == torch.bfloat16 and _GEMM_BACKEND != "cublas" and gate_up.dim() == 2 and gate_up.shape[-1] % 16 == 0
          and not _small_or_odd(gate_up[:, : gate_up.shape[-1] // 2], weight) and not _fp8(weight))
    if not ok:
        return linear(swiglu(gate_up), weight)
    return _SwiGLULinear.apply(gate_up, weight)


# ------------------------------------------------------------------------------- qkv prep
class _QKVNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, qw, kw, cos, sin, n_q, n_kv, D, eps, offset, gated):
        qkvc = qkv.contiguous()
        outs = _C.qkv_norm_rope_fwd(qkvc, n_q, n_kv, D, qw, kw, cos, sin, eps, offset, gated)
        q, k, v, rstd = outs[:4]
        gate = outs[4] if gated else None
        ctx.save_for_backward(qkvc, qw, kw, cos, sin, rstd)
        ctx.cfg = (n_q, n_kv, D, offset, gated)
        _tick()
        if gated:
            return q, k, v, gate
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv, dgate=None):
        qkv, qw, kw, cos, sin, rstd = ctx.saved_tensors
        n_q, n_kv, D, offset, gated = ctx.cfg
        dqkv, dqw, dkw = _C.qkv_norm_rope_bwd(dq.contiguous(), dk.contiguous(), dv.contiguous(),
                                              dgate.contiguous() if gated else None, qkv, qw, kw, cos, sin, rstd,
                                              n_q, n_kv, D, offset, gated)
        _tick(2)
        if qw is None:
            return (dqkv,) + (None,) * 10
        return dqkv, dqw.to(qw.dtype), dkw.to(kw.dtype), None, None, None, None, None, None, None, None


def qkv_norm_rope(qkv, n_q, n_kv, head_dim, q_weight, k_weight, cos, sin, eps=1e-6, offset=False, gated=False):
    cos = cos.float().contiguous()
    sin = sin.float().contiguous()
    out = _QKVNormRope.apply(qkv, q_weight, k_weight, cos, sin, n_q, n_kv, head_dim, eps, offset, gated)
    if gated:
        return out
    return out[0], out[1], out[2], None


class _RopeGeneric(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, d_out):
        ctx.save_for_backward(cos, sin)
        ctx.d = x.shape[-1]
        _tick()
        return _C.rope_generic(x, cos, sin, False, d_out)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        _tick()
        return _C.rope_generic(dy[..., :ctx.d], cos, sin, True, ctx.d), None, None, None


def rope_vision(q, k, cos, sin, pad_to=None):
    """``pad_to``: emit ``[S, H, pad_to]`` with zeros behind the rotated channels (the attention kernel's tile width)."""
    cos, sin = cos.float().contiguous(), sin.float().contiguous()
    d_out = pad_to or q.shape[-1]
    return _RopeGeneric.apply(q, cos, sin, d_out), _RopeGeneric.apply(k, cos, sin, d_out)


# ------------------------------------------------------------------------------- attention
def _pad_heads(t, d_to):
    if t.shape[-1] == d_to:
        return t.contiguous()
    return torch.nn.functional.pad(t, (0, d_to - t.shape[-1]))


def _heads_in_place(t):
    """``[T, H, d]`` as the attention kernels' tensor maps can read it: unit channel stride, 16-byte aligned head and token
    strides and base (a slice of a fused projection qualifies); anything else is copied."""
    if t.stride(2) == 1 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _AttentionVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal, scale):
        q, k, v = _heads_in_place(q), _heads_in_place(k), _heads_in_place(v)
        o, lse = _C.attn_fwd(q, k, v, cu_seqlens, max_seqlen, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.cfg = (max_seqlen, causal, scale)
        _tick()
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu = ctx.saved_tensors
        max_seqlen, causal, scale = ctx.cfg
        dq, dk, dv = _C.attn_bwd(do.contiguous(), q, k, v, o, lse, cu, max_seqlen, causal, scale)
        _tick(3)
        return dq, dk, dv, None, None, None, None


def attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal=True, scale=None):
    """Varlen attention over packed rows.  Head sizes that are a multiple of 8 up to 128 run as they are (the kernels' tiles
    are 64 or 128 wide and TMA zero-fills the rest), 256 on the single-tile kernels; sizes in between are zero-padded."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if q.dtype != torch.bfloat16:
        return ref.attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale)
    if not hasattr(_C, "attn_fwd"):
        raise RuntimeError("the attention kernel is not part of this build of the extension")
    cu = cu_seqlens.to(torch.int32)
    if D == 256 or (D <= 128 and D % 8 == 0):
        if D == 256:
            q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        return _AttentionVarlen.apply(q, k, v, cu, int(max_seqlen), bool(causal), float(scale))
    if D < 128:
        pad = (D + 7) // 8 * 8
        o = _AttentionVarlen.apply(_pad_heads(q, pad), _pad_heads(k, pad), _pad_heads(v, pad), cu, int(max_seqlen), bool(causal), float(scale))
        return o[..., :D]
    if D < 256:
        o = _AttentionVarlen.apply(_pad_heads(q, 256), _pad_heads(k, 256), _pad_heads(v, 256), cu, int(max_seqlen), bool(causal), float(scale))
        return o[..., :D]
    raise NotImplementedError(f"attention_varlen: head size {D} is beyond the tcgen05 kernels (up to 128, 256 and what pads to them)")


def dsa_attention(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk, scale=None, cu_host=None):
    from .dsa_cuda import dsa_attention_cuda

    return dsa_attention_cuda(q, k, v, idx_q, idx_k, idx_w, cu_seqlens, topk, scale, cu_host)


# ------------------------------------------------------------------------------- loss
class _LinearCrossEntropy(torch.autograd.Function):
    """Chunked ``cross_entropy(h W^T)``: per chunk of rows one logits GEMM, one fused
    softmax/loss/gradient kernel that overwrites the logits with d(logits), then the two
    gradient GEMMs.  Gradients are produced in the forward pass (scaled by ``grad_scale``),
    so the ``[T, V]`` logits never exist and nothing of size V is saved for backward."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, chunk, ignore_index, grad_scale):
        T, H = hidden.shape
        V = weight.shape[0]
        hidden = _as_gemm_operand(hidden)
        weight_c = _as_gemm_operand(weight)
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh = torch.empty_like(hidden) if need_dh else None
        dw = torch.zeros(V, H, dtype=torch.float32, device=hidden.device) if need_dw else None
        losses = torch.empty(T, dtype=torch.float32, device=hidden.device)
        targets = targets.contiguous()
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            hc = hidden[s:e]
            logits = _gemm(hc, weight_c)  # [C, V]
            losses[s:e] = _C.ce_fwd_bwd_(logits, targets[s:e], grad_scale, ignore_index)
            _tick()
            if need_dh:
                _gemm(logits, weight_c, b_mn=True, out=dh[s:e])  # dH = dL . W
            if need_dw:
                _gemm(logits, hc, a_mn=True, b_mn=True, out=dw, accumulate=True)  # dW += dL^T . H
        ctx.save_for_backward(dh, dw)
        ctx.w_dtype = weight.dtype
        n_valid = (targets != ignore_index).sum()
        ctx.mark_non_differentiable(n_valid)
        return losses.sum(), n_valid

    @staticmethod
    def backward(ctx, g_loss, _g_n):
        dh, dw = ctx.saved_tensors
        # the kernels already applied grad_scale; g_loss is the upstream scalar on the *sum* loss
        if dh is not None:
            dh = dh * g_loss.to(dh.dtype)
        if dw is not None:
            dw = (dw * g_loss).to(ctx.w_dtype)
        return dh, dw, None, None, None, None


def linear_cross_entropy(hidden, weight, targets, chunk=1024, ignore_index=-100, grad_scale: float = 1.0):
    if hidden.dtype != torch.bfloat16 or not _tma_ok(hidden, weight) or weight.shape[0] % 8:
        return ref.linear_cross_entropy(hidden, weight, targets, chunk, ignore_index)
    return _LinearCrossEntropy.apply(hidden, weight, targets, int(chunk), int(ignore_index), float(grad_scale))


# ------------------------------------------------------------------------------- GDN
class _ConvSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, seq_idx):
        wc = w.contiguous()
        ctx.save_for_backward(x, wc, seq_idx)
        _tick()
        return _C.conv1d_silu_fwd(x, wc, seq_idx)

    @staticmethod
    def backward(ctx, dy):
        x, w, seq_idx = ctx.saved_tensors
        dx, dw = _C.conv1d_silu_bwd(dy if dy.stride(-1) == 1 else dy.contiguous(), x, w, seq_idx)
        _tick(2)
        return dx, dw.to(w.dtype), None


def causal_conv1d_silu(x, weight, seq_idx):
    if x.dtype != torch.bfloat16 or weight.shape[1] != 4 or x.shape[1] % 8 or x.stride(0) % 8 or x.stride(1) != 1:
        return ref.causal_conv1d_silu(x, weight, seq_idx)
    return _ConvSilu.apply(x, weight, seq_idx)


class _GdnGates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, A_log, dt_bias):
        Af, df = A_log.float().contiguous(), dt_bias.float().contiguous()
        g, beta = _C.gdn_gates_fwd(a, b, Af, df)
        ctx.save_for_backward(a, b, Af, df)
        ctx.dtypes = (A_log.dtype, dt_bias.dtype)
        _tick()
        return g, beta

    @staticmethod
    def backward(ctx, dg, dbeta):
        a, b, Af, df = ctx.saved_tensors
        da, db, dA, ddt = _C.gdn_gates_bwd(dg, dbeta, a, b, Af, df)
        _tick(2)
        return da, db, dA.to(ctx.dtypes[0]), ddt.to(ctx.dtypes[1])


def gdn_gates(a, b, A_log, dt_bias):
    ok = (a.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
          and a.stride(0) == b.stride(0) and a.shape[1] <= 256)
    if not ok:
        g = -A_log.float().exp() * torch.nn.functional.softplus(a.float() + dt_bias.float())
        return g, torch.sigmoid(b.float()).to(b.dtype)
    return _GdnGates.apply(a, b, A_log, dt_bias)


def gdn_scan(x1, x2, e, decay, ext, ranges, reverse, head_major=False):
    """The chunk-to-chunk scan of :mod:`.gdn_scan` as one tcgen05 kernel launch (``csrc/gdn_scan_sm100.cu``):
    bf16 operands ``[chunks, heads, 64, 128]`` (``head_major``: ``[heads, chunks, 64, 128]``).  Other shapes run the
    tensor-operation loop."""
    if x1.dtype == torch.bfloat16 and x1.shape[2:] == (64, 128) and e.shape[3] == 128:
        y, states = _C.gdn_scan(x1, x2, e, decay.float().contiguous(), ext.to(torch.bfloat16) if ext is not None else None,
                                ranges[2], reverse, head_major)
        _tick()
        return y, states
    from .gdn_scan import scan_torch

    return scan_torch(x1, x2, e, decay, ext, ranges[0], ranges[1], reverse, head_major)


def gated_delta_rule(q, k, v, g, beta, cu_seqlens, scale=None, chunk=64, cu_host=None):
    if cu_host is None:
        cu_host = cu_seqlens.tolist()  # one device sync; pass cu_host to avoid it
    if q.shape[-1] == 128 and v.shape[-1] == 128 and chunk == 64 and os.environ.get("VLMT_GDN_SCAN", "1") != "0":
        from .gdn_scan import gated_delta_rule_scan

        return gated_delta_rule_scan(q, k, v, g, beta, cu_host, scale, chunk)
    # other head sizes: the recurrence as batched library operations, one step per chunk position
    from .gdn_batched import gated_delta_rule_batched

    return gated_delta_rule_batched(q, k, v, g, beta, cu_host, scale, chunk)


# ------------------------------------------------------------------------------- MoE
def moe_router(logits, top_k, renorm=True):
    from .moe_cuda import moe_router_cuda

    return moe_router_cuda(logits, top_k, renorm)


def moe_experts(x, gate_up, down, weights, experts):
    from .moe_cuda import moe_experts_cuda

    return moe_experts_cuda(x, gate_up, down, weights, experts)


# ------------------------------------------------------------------------------- rows
class _RowsUpdate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, index, src, add):
        out = x.clone()
        _C.rows_update(out, index, src.contiguous().to(x.dtype), add)
        ctx.save_for_backward(index)
        ctx.add = add
        _tick()
        return out

    @staticmethod
    def backward(ctx, dout):
        (index,) = ctx.saved_tensors
        dout = dout.contiguous()
        dsrc = _C.rows_gather(dout, index)
        _tick()
        if ctx.add:
            return dout, None, dsrc, None
        dx = dout.clone()
        _C.rows_update(dx, index, torch.zeros_like(dsrc), False)
        return dx, None, dsrc, None


def scatter_rows(x, index, src):
    if x.dtype != torch.bfloat16 or x.shape[-1] % 8:
        return ref.scatter_rows(x, index, src)
    return _RowsUpdate.apply(x, index, src, False)


def add_rows(x, index, src):
    if x.dtype != torch.bfloat16 or x.shape[-1] % 8:
        return ref.add_rows(x, index, src)
    return _RowsUpdate.apply(x, index, src, True)


# ------------------------------------------------------------------------------- optimizer
def adamw_step_(grad, master, exp_avg, exp_avg_sq, param, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                zero_grad=False):
    """``zero_grad``: clear ``grad`` after it has been consumed (no separate memset before the next step)."""
    _C.adamw_(grad, master, exp_avg, exp_avg_sq, param, lr, beta1, beta2, eps, weight_decay, step, grad_scale, zero_grad)
    _tick()


def memset_zero_(t):
    """Clear a contiguous tensor with the driver's memset on the current stream (write-only, at memory speed)."""
    _C.memset_zero_(t)


def sumsq_(x, out):
    _C.sumsq_(x, out)
    _tick()
