"""FP8 training of linear layers: tensor-wise dynamic scaling, e4m3 for activations and weights, e5m2 for output
gradients, fp32 accumulation, bf16 results.

The capability mirrors the reference's ``apply_float8`` hook (reference: train/infra.py:139-153, torchao's
``convert_to_float8_training`` with a filter that skips the vision tower and dimensions that are not multiples of 16).
Here the three GEMMs of a linear layer run on the FP8 tensor cores (``fp8_sm100.cu``: ``tcgen05.mma kind::f8f6f4``).
That kernel takes K-major operands only, so the quantisation kernel writes a matrix and its transpose in one pass:

    forward            y  = x8 . w8^T          x8 [T, K],  w8 [N, K]
    input gradient     dx = dy8 . (w8^T)^T     dy8 [T, N], w8^T [K, N]
    weight gradient    dw = dy8^T . (x8^T)^T   dy8^T [N, T], x8^T [K, T]   (added into the gradient bucket in place)

``x8^T`` (one byte per element) is what is kept for backward instead of the bf16 activation.  On CPU the same arithmetic
is emulated with torch's float8 dtypes, which is also the oracle of the GPU tests.
"""
from __future__ import annotations

import torch

E4M3, E5M2 = 0, 1
_MAX = {E4M3: 448.0, E5M2: 57344.0}
_DTYPE = {E4M3: torch.float8_e4m3fn, E5M2: torch.float8_e5m2}

CALLS = {"linear": 0}  # FP8 linears run (forward calls); tests read it to see that the marked weights took this path


def marked(weight) -> bool:
    return bool(getattr(weight, "_vlmt_fp8", False))


def quantize_ref(x: torch.Tensor, fmt: int):
    """Plain PyTorch form of the quantisation kernel: ``(q as float8, inverse scale)``."""
    amax = x.detach().abs().amax().float().clamp_min(1e-12)
    scale = _MAX[fmt] / amax
    q = (x.detach().float() * scale).clamp(-_MAX[fmt], _MAX[fmt]).to(_DTYPE[fmt])
    return q, amax / _MAX[fmt]


class _LinearFp8Ref(torch.autograd.Function):
    """The FP8 linear in plain PyTorch (any device): quantise, multiply in fp32, rescale."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1])
        xq, sx = quantize_ref(x2, E4M3)
        wq, sw = quantize_ref(w, E4M3)
        y = (xq.float() @ wq.float().t()) * (sx * sw)
        if b is not None:
            y = y + b.float()
        ctx.save_for_backward(xq, wq, sx, sw)
        ctx.has_bias, ctx.in_shape, ctx.dtype = b is not None, x.shape, x.dtype
        return y.to(x.dtype).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xq, wq, sx, sw = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dq, sd = quantize_ref(dy2, E5M2)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = ((dq.float() @ wq.float()) * (sd * sw)).to(ctx.dtype).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw = ((dq.float().t() @ xq.float()) * (sd * sx)).to(ctx.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear_ref(x, weight, bias=None):
    return _LinearFp8Ref.apply(x, weight, bias)


def usable(x, weight) -> bool:
    """Shapes the FP8 kernels take: bf16, both dimensions multiples of 16, rows a multiple of 16."""
    rows = x.numel() // max(1, x.shape[-1])
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2
            and weight.shape[0] % 16 == 0 and weight.shape[1] % 16 == 0 and rows % 16 == 0 and rows > 0)


class _LinearFp8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b):
        from . import cuda as cu

        C = cu._C
        x2 = cu._as_gemm_operand(x.reshape(-1, x.shape[-1]))
        wc = cu._as_gemm_operand(w)
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        x8, x8t, rx = C.fp8_quantize(x2, E4M3, True, need_dw)
        w8, w8t, rw = C.fp8_quantize(wc, E4M3, True, need_dx)
        y = torch.empty(x2.shape[0], w.shape[0], dtype=torch.bfloat16, device=x.device)
        C.gemm_fp8(x8, w8, y, rx, rw, E4M3, E4M3, False)
        cu._tick(5)
        if b is not None:
            y = y + b
        ctx.save_for_backward(x8t, w8t, rx, rw)
        ctx.w_param = cu._grad_target(w)
        ctx.has_bias, ctx.in_shape, ctx.w_shape = b is not None, x.shape, tuple(w.shape)
        CALLS["linear"] += 1
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import cuda as cu

        C = cu._C
        x8t, w8t, rx, rw = ctx.saved_tensors
        dy2 = cu._as_gemm_operand(dy.reshape(-1, dy.shape[-1]))
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        d8, d8t, rd = C.fp8_quantize(dy2, E5M2, need_dx, need_dw)
        cu._tick(2)
        dx = dw = db = None
        if need_dx:
            dx = torch.empty(dy2.shape[0], ctx.w_shape[1], dtype=torch.bfloat16, device=dy.device)
            C.gemm_fp8(d8, w8t, dx, rd, rw, E5M2, E4M3, False)
            cu._tick()
            dx = dx.view(ctx.in_shape)
        if need_dw:
            param = ctx.w_param
            g = param.grad if param is not None else None
            if (g is not None and g.dtype == torch.bfloat16 and g.dim() == 2 and tuple(g.shape) == ctx.w_shape and g.stride(1) == 1
                    and g.stride(0) % 8 == 0 and g.data_ptr() % 16 == 0):
                # added into the optimizer's gradient bucket by the GEMM's epilogue; autograd has nothing to accumulate
                C.gemm_fp8(d8t, x8t, g, rd, rx, E5M2, E4M3, True)
                ready = getattr(param, "_vlmt_grad_ready", None)
                if ready is not None:
                    ready(param)
            else:
                dw = torch.empty(ctx.w_shape, dtype=torch.bfloat16, device=dy.device)
                C.gemm_fp8(d8t, x8t, dw, rd, rx, E5M2, E4M3, False)
            cu._tick()
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = cu._colsum(dy2).to(dy.dtype)
        return dx, dw, db


def linear(x, weight, bias=None):
    """``x W^T (+ b)`` with the three GEMMs in FP8; shapes the kernels do not take use the emulation."""
    if usable(x, weight):
        return _LinearFp8.apply(x, weight, bias)
    CALLS["linear"] += 1
    return linear_ref(x, weight, bias)
