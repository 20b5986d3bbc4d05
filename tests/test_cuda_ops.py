"""Numerics of every CUDA kernel against the plain-PyTorch fp32 statement of the same op.
All tests here need a B200; they are skipped on machines without CUDA."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from vlm_training_b200 import ops
from vlm_training_b200.ops import reference as ref

DEV = "cuda"


def _cu():
    from vlm_training_b200.ops import cuda as cu

    return cu


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV) * scale).to(dtype)


def _close(got, want, atol, rtol, what=""):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4g}, max ref {want.abs().max().item():.4g}, " \
                                     f"frac bad {(err > tol).float().mean().item():.4g}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (1000, 1152, 1536), (384, 4304, 1152), (8, 16, 8),
                                   (2048, 4096, 4096), (130, 136, 72)])
def test_gemm_forward_layout(M, N, K):
    cu = _cu()
    a, b = _rand(M, K), _rand(N, K)
    got = cu._gemm(a, b)
    want = a.float() @ b.float().t()
    _close(got, want, atol=0.05 * math.sqrt(K) / 8, rtol=2e-2, what=f"gemm KK {M}x{N}x{K}")
    cu.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (1000, 1152, 4304), (777, 136, 72)])
def test_gemm_wgrad_adds_into_bf16_gradient(M, N, K):
    """bf16 accumulate: the slabs are added by TMA reduce-adds; the previous content of D must survive."""
    cu = _cu()
    dy, x = _rand(M, N), _rand(M, K)
    before = _rand(N, K, scale=3.0)
    acc = before.clone()
    cu._gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True)
    want = before.float() + dy.float().t() @ x.float()
    _close(acc, want, atol=0.05 * math.sqrt(M) / 8 + 0.05, rtol=2e-2, what="wgrad bf16 acc")
    cu.check_status()


def test_linear_wgrad_in_place_into_tagged_gradient():
    """A parameter tagged by the optimizer engine gets its weight gradient added into ``.grad`` by the GEMM itself:
    autograd sees ``None``, the ready hook fires once, and activation checkpointing does not change that."""
    from torch.utils.checkpoint import checkpoint

    cu = _cu()
    torch.manual_seed(3)
    lin = torch.nn.Linear(256, 384, bias=False, device=DEV, dtype=torch.bfloat16)
    norm_w = torch.nn.Parameter(torch.ones(256, device=DEV, dtype=torch.bfloat16))
    flat = torch.zeros(384 * 256 + 8, device=DEV, dtype=torch.bfloat16)
    w = lin.weight
    w.grad = flat[8:].view(384, 256)
    w._vlmt_grad_in_place = True
    fired = []
    w._vlmt_grad_ready = lambda p: fired.append(id(p))
    x = _rand(512, 256).requires_grad_()
    g = _rand(512, 384, scale=0.1)
    want = g.float().t() @ x.detach().float()

    def check(times):
        _close(flat[8:].view(384, 256), times * want, atol=0.08 * times, rtol=2e-2, what=f"in-place wgrad x{times}")
        assert float(flat[:8].abs().sum()) == 0.0

    ops.linear(x, w).backward(g)
    assert fired == [id(w)]
    check(1)
    checkpoint(lambda t: ops.linear(t, w), x, use_reentrant=False).backward(g)     # second micro-batch: accumulates
    assert fired == [id(w)] * 2
    check(2)
    y = ops.rms_norm_linear(x, norm_w, w, 1e-6)
    y.backward(g)
    assert len(fired) == 3 and norm_w.grad is not None
    assert x.grad is not None
    cu.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (1000, 1152, 4304), (2048, 4096, 12288)])
def test_gemm_dgrad_wgrad_layouts(M, N, K):
    cu = _cu()
    # dgrad: dX[M,K] = dY[M,N] . W[N,K]   (A K-major, B stored [contraction, out])
    dy, w, x = _rand(M, N), _rand(N, K), _rand(M, K)
    got = cu._gemm(dy, w, b_mn=True)
    _close(got, dy.float() @ w.float(), atol=0.05 * math.sqrt(N) / 8, rtol=2e-2, what="dgrad")
    # wgrad: dW[N,K] = dY^T . X   (both stored [contraction, out])
    got = cu._gemm(dy, x, a_mn=True, b_mn=True)
    _close(got, dy.float().t() @ x.float(), atol=0.05 * math.sqrt(M) / 8, rtol=2e-2, what="wgrad")
    # fp32 accumulate-into
    acc = torch.ones(N, K, device=DEV)
    cu._gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True)
    _close(acc, 1.0 + dy.float().t() @ x.float(), atol=0.05 * math.sqrt(M) / 8, rtol=2e-2, what="wgrad acc")
    cu.check_status()


def test_gemm_bias_and_repeatability():
    cu = _cu()
    a, b, bias = _rand(512, 1152), _rand(3456, 1152), _rand(3456)
    got = cu._gemm(a, b, bias=bias)
    _close(got, a.float() @ b.float().t() + bias.float(), atol=0.3, rtol=2e-2, what="bias")
    assert torch.equal(got, cu._gemm(a, b, bias=bias)), "two runs differ"


def test_linear_autograd_matches_torch():
    x = _rand(300, 256, scale=0.5).requires_grad_()
    w = _rand(512, 256, scale=0.1).requires_grad_()
    b = _rand(512, scale=0.1).requires_grad_()
    y = ops.linear(x, w, b)
    g = _rand(300, 512)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    _close(y, yr, 0.05, 2e-2, "y")
    _close(x.grad, xr.grad, 0.1, 2e-2, "dx")
    _close(w.grad, wr.grad, 0.3, 2e-2, "dw")
    _close(b.grad, br.grad, 0.3, 2e-2, "db")


@pytest.mark.parametrize("offset", [False, True])
@pytest.mark.parametrize("D", [128, 4096, 1152, 8192])
def test_rms_norm_fwd_bwd(D, offset):
    x = _rand(777, D).requires_grad_()
    w = _rand(D, scale=0.3).requires_grad_()
    y = ops.rms_norm(x, w, 1e-6, offset)
    g = _rand(777, D)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rms_norm(xr, wr, 1e-6, offset)
    yr.backward(g.float())
    _close(y, yr, 0.02, 1e-2, "y")
    _close(x.grad, xr.grad, 0.03, 2e-2, "dx")
    _close(w.grad, wr.grad, 0.5, 2e-2, "dw")


def test_add_rms_norm_fwd_bwd():
    D = 512
    x, r = _rand(300, D).requires_grad_(), _rand(300, D).requires_grad_()
    w = _rand(D, scale=0.3).requires_grad_()
    y, s = ops.add_rms_norm(x, r, w, 1e-6, False)
    gy, gs = _rand(300, D), _rand(300, D)
    torch.autograd.backward([y, s], [gy, gs])
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    sr = xr + rr
    yr = ref.rms_norm(sr, wr, 1e-6, False)
    torch.autograd.backward([yr, sr], [gy.float(), gs.float()])
    _close(y, yr, 0.03, 2e-2, "y")
    _close(s, sr, 0.03, 1e-2, "sum")
    _close(x.grad, xr.grad, 0.05, 2e-2, "dx")
    _close(r.grad, rr.grad, 0.05, 2e-2, "dres")
    _close(w.grad, wr.grad, 0.5, 2e-2, "dw")


@pytest.mark.parametrize("D", [1152, 4608, 1024, 1032, 776, 768])
def test_layer_norm_fwd_bwd(D):
    x = _rand(500, D).requires_grad_()
    w, b = _rand(D, scale=0.5).requires_grad_(), _rand(D, scale=0.5).requires_grad_()
    y = ops.layer_norm(x, w, b, 1e-6)
    g = _rand(500, D)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (D,), wr, br, 1e-6)
    yr.backward(g.float())
    _close(y, yr, 0.03, 1e-2, "y")
    _close(x.grad, xr.grad, 0.05, 2e-2, "dx")
    _close(w.grad, wr.grad, 0.5, 2e-2, "dw")
    _close(b.grad, br.grad, 0.5, 2e-2, "db")


def test_rms_norm_gated_fwd_bwd():
    D = 128
    x, z = _rand(1000, D).requires_grad_(), _rand(1000, D).requires_grad_()
    w = _rand(D, scale=0.5).requires_grad_()
    y = ops.rms_norm_gated(x, z, w, 1e-6)
    g = _rand(1000, D)
    y.backward(g)
    xr, zr, wr = (t.detach().float().requires_grad_() for t in (x, z, w))
    yr = ref.rms_norm_gated(xr, zr, wr, 1e-6)
    yr.backward(g.float())
    _close(y, yr, 0.03, 2e-2, "y")
    _close(x.grad, xr.grad, 0.05, 2e-2, "dx")
    _close(z.grad, zr.grad, 0.05, 2e-2, "dz")
    _close(w.grad, wr.grad, 0.6, 2e-2, "dw")


def test_swiglu_sigmoid_mul_gelu():
    gu = _rand(257, 2 * 768).requires_grad_()
    y = ops.swiglu(gu)
    g = _rand(257, 768)
    y.backward(g)
    gr = gu.detach().float().requires_grad_()
    a, b = gr.chunk(2, -1)
    yr = torch.nn.functional.silu(a) * b
    yr.backward(g.float())
    _close(y, yr, 0.02, 1e-2, "swiglu")
    _close(gu.grad, gr.grad, 0.03, 2e-2, "swiglu grad")

    x, gt = _rand(100, 512).requires_grad_(), _rand(100, 512).requires_grad_()
    y = ops.sigmoid_mul(x, gt)
    g = _rand(100, 512)
    y.backward(g)
    xr, gtr = x.detach().float().requires_grad_(), gt.detach().float().requires_grad_()
    (xr * torch.sigmoid(gtr)).backward(g.float())
    _close(x.grad, xr.grad, 0.02, 2e-2, "sigmul dx")
    _close(gt.grad, gtr.grad, 0.02, 2e-2, "sigmul dgate")

    cu = _cu()
    for approx in ("tanh", "none"):
        x = _rand(64, 1024).requires_grad_()
        y = cu.gelu(x, approx)
        y.backward(g := _rand(64, 1024))
        xr = x.detach().float().requires_grad_()
        yr = torch.nn.functional.gelu(xr, approximate=approx)
        yr.backward(g.float())
        _close(y, yr, 0.02, 1e-2, f"gelu {approx}")
        _close(x.grad, xr.grad, 0.03, 2e-2, f"gelu grad {approx}")


@pytest.mark.parametrize("D,R,gated,offset", [(128, 128, False, False), (256, 64, True, True), (64, 64, False, False),
                                              (32, 32, False, False), (64, 16, True, True)])
def test_qkv_norm_rope_fwd_bwd(D, R, gated, offset):
    T, n_q, n_kv = 193, 4, 2
    W = (n_q * (2 if gated else 1) + 2 * n_kv) * D
    qkv = _rand(T, W).requires_grad_()
    qw, kw = _rand(D, scale=0.3).requires_grad_(), _rand(D, scale=0.3).requires_grad_()
    ang = torch.rand(T, R // 2, device=DEV) * 6.28
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos(), emb.sin()
    outs = ops.qkv_norm_rope(qkv, n_q, n_kv, D, qw, kw, cos, sin, 1e-6, offset, gated)
    grads = [_rand(*o.shape) for o in outs if o is not None]
    torch.autograd.backward([o for o in outs if o is not None], grads)
    import vlm_training_b200.ops as O

    qkvr, qwr, kwr = (t.detach().float().requires_grad_() for t in (qkv, qw, kw))
    O._FORCE_REF = True
    try:
        outs_r = ops.qkv_norm_rope(qkvr, n_q, n_kv, D, qwr, kwr, cos, sin, 1e-6, offset, gated)
    finally:
        O._FORCE_REF = False
    torch.autograd.backward([o for o in outs_r if o is not None], [g.float() for g in grads])
    for name, a, b in zip("qkvg", outs, outs_r):
        if a is not None:
            _close(a, b, 0.03, 2e-2, name)
    _close(qkv.grad, qkvr.grad, 0.06, 3e-2, "dqkv")
    _close(qw.grad, qwr.grad, 0.8, 3e-2, "dqw")
    _close(kw.grad, kwr.grad, 0.8, 3e-2, "dkw")


def test_rope_vision_fwd_bwd():
    S, H, D = 300, 4, 72
    qkv = _rand(S, 3, H, D).requires_grad_()
    ang = torch.rand(S, D // 2, device=DEV) * 6.28
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos(), emb.sin()
    q, k, v = qkv.unbind(1)
    qo, ko = ops.rope_vision(q, k, cos, sin)
    gq, gk = _rand(S, H, D), _rand(S, H, D)
    torch.autograd.backward([qo, ko], [gq, gk])
    qr = qkv.detach().float().requires_grad_()
    q2, k2, _ = qr.unbind(1)
    qo_r, ko_r = ref.apply_rope(q2, cos, sin), ref.apply_rope(k2, cos, sin)
    torch.autograd.backward([qo_r, ko_r], [gq.float(), gk.float()])
    _close(qo, qo_r, 0.02, 1e-2, "q")
    _close(ko, ko_r, 0.02, 1e-2, "k")
    _close(qkv.grad, qr.grad, 0.03, 2e-2, "dqkv")


def test_gdn_gates_and_conv():
    T, H, C = 500, 16, 512
    proj = _rand(T, C + 2 * H).requires_grad_()
    A_log, dt_bias = _rand(H, scale=0.5).requires_grad_(), _rand(H).requires_grad_()
    x, a, b = proj.split([C, H, H], -1)
    g, beta = ops.gdn_gates(a, b, A_log, dt_bias)
    cu_seq = torch.tensor([0, 100, 101, 350, 500], device=DEV, dtype=torch.int32)
    seq_idx = ref.seq_idx_from_cu(cu_seq, T)
    w = _rand(C, 4, scale=0.5).requires_grad_()
    y = ops.causal_conv1d_silu(x, w, seq_idx)
    gg, gb, gy = torch.randn(T, H, device=DEV), _rand(T, H), _rand(T, C)
    torch.autograd.backward([g, beta, y], [gg, gb, gy])

    pr, Ar, dr, wr = (t.detach().float().requires_grad_() for t in (proj, A_log, dt_bias, w))
    xr, ar, br = pr.split([C, H, H], -1)
    g_r = -Ar.exp() * torch.nn.functional.softplus(ar + dr)
    beta_r = torch.sigmoid(br)
    y_r = ref.causal_conv1d_silu(xr, wr, seq_idx)
    torch.autograd.backward([g_r, beta_r, y_r], [gg, gb.float(), gy.float()])
    _close(g, g_r, 0.02, 1e-2, "g")
    _close(beta, beta_r, 0.01, 1e-2, "beta")
    _close(y, y_r, 0.03, 2e-2, "conv y")
    _close(proj.grad, pr.grad, 0.06, 3e-2, "dproj")
    _close(w.grad, wr.grad, 1.0, 3e-2, "dconv w")
    _close(A_log.grad, Ar.grad, 2.0, 3e-2, "dA_log")
    _close(dt_bias.grad, dr.grad, 2.0, 3e-2, "ddt_bias")


def test_rows_scatter_add():
    x = _rand(1000, 256).requires_grad_()
    idx = torch.randperm(1000, device=DEV)[:300].sort().values
    src = _rand(300, 256).requires_grad_()
    for fn, rfn in ((ops.scatter_rows, ref.scatter_rows), (ops.add_rows, ref.add_rows)):
        x.grad = src.grad = None
        y = fn(x, idx, src)
        g = _rand(1000, 256)
        y.backward(g)
        xr, sr = x.detach().float().requires_grad_(), src.detach().float().requires_grad_()
        yr = rfn(xr, idx, sr)
        yr.backward(g.float())
        _close(y, yr, 0.02, 1e-2, "y")
        _close(x.grad, xr.grad, 1e-3, 1e-3, "dx")
        _close(src.grad, sr.grad, 1e-3, 1e-3, "dsrc")


@pytest.mark.parametrize("T,H,V,chunk", [(700, 256, 5000, 256), (1024, 512, 151936, 512)])
def test_linear_cross_entropy(T, H, V, chunk):
    h = _rand(T, H, scale=0.5).requires_grad_()
    w = _rand(V, H, scale=0.05).requires_grad_()
    tgt = torch.randint(0, V, (T,), device=DEV)
    tgt[::7] = -100
    loss_sum, n = ops.linear_cross_entropy(h, w, tgt, chunk)
    (loss_sum / n).backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logits = (hr @ wr.t()).to(torch.bfloat16).float()  # the kernel sees bf16 logits
    lr = torch.nn.functional.cross_entropy(logits, tgt, ignore_index=-100)
    lr.backward()
    assert int(n) == int((tgt != -100).sum())
    assert abs((loss_sum / n).item() - lr.item()) < 2e-2, ((loss_sum / n).item(), lr.item())
    _close(h.grad, hr.grad, 2e-4, 5e-2, "dh")
    _close(w.grad, wr.grad, 2e-4, 5e-2, "dw")


def test_adamw_matches_torch():
    cu = _cu()
    n = 100_003
    p0 = torch.randn(n, device=DEV)
    master, m, v = p0.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    param = p0.to(torch.bfloat16)
    pr = p0.clone().requires_grad_()
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(torch.bfloat16)
        cu.adamw_step_(g, master, m, v, param, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
        pr.grad = g.float()
        opt.step()
    torch.testing.assert_close(master, pr.detach(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(param.float(), pr.detach().to(torch.bfloat16).float(), atol=1e-2, rtol=1e-2)


def test_adamw_clears_gradient_and_handles_unaligned_ranges():
    """``zero_grad=True`` leaves the consumed gradient range at zero; a range that does not start on a 16-byte boundary
    takes the scalar path and must give the same update as the vector path."""
    cu = _cu()
    n = 40_000
    big = torch.randn(n + 8, device=DEV)
    g_all = torch.randn(n + 8, device=DEV).to(torch.bfloat16)
    outs = []
    for off in (0, 1):   # aligned / unaligned views of the same data
        master = big[off:off + n].clone()
        m, v = torch.zeros(n + 8, device=DEV)[off:off + n], torch.zeros(n + 8, device=DEV)[off:off + n]
        gbuf = g_all.clone()
        g = gbuf[off:off + n]
        pbuf = torch.zeros(n + 8, device=DEV, dtype=torch.bfloat16)
        mbuf = torch.empty(n + 8, device=DEV)
        mview = mbuf[off:off + n]
        mview.copy_(master)
        cu.adamw_step_(g, mview, m, v, pbuf[off:off + n], 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 0.5, zero_grad=True)
        assert float(g.float().abs().max()) == 0.0
        if off == 1:
            assert float(gbuf[0].float().abs()) == float(g_all[0].float().abs())   # outside the range: untouched
        outs.append((mview.clone(), g_all[off:off + n].clone(), big[off:off + n].clone()))
    for mview, g_in, p0 in outs:
        gf = g_in.float() * 0.5
        want = p0 * (1 - 1e-2 * 0.1) - 1e-2 * ((0.1 * gf) / (1 - 0.9)) / (((0.05 * gf * gf) / (1 - 0.95)).sqrt() + 1e-8)
        torch.testing.assert_close(mview, want, atol=1e-5, rtol=1e-5)


def test_norm_linear_and_swiglu_linear_match_unfused():
    """The memory-saving fused forms must give the same values and gradients as the unfused sequence."""
    T, H, N, I = 300, 512, 768, 1024
    x, r = _rand(T, H).requires_grad_(), _rand(T, H).requires_grad_()
    nw, w = _rand(H, scale=0.3).requires_grad_(), _rand(N, H, scale=0.05).requires_grad_()
    y, s = ops.rms_norm_linear(x, nw, w, 1e-6, False, r)
    gy, gs = _rand(T, N), _rand(T, H)
    torch.autograd.backward([y, s], [gy, gs])
    xr, rr, nwr, wr = (t.detach().float().requires_grad_() for t in (x, r, nw, w))
    sr = xr + rr
    yr = torch.nn.functional.linear(ref.rms_norm(sr, nwr, 1e-6, False), wr)
    torch.autograd.backward([yr, sr], [gy.float(), gs.float()])
    _close(y, yr, 0.05, 2e-2, "y")
    _close(x.grad, xr.grad, 0.05, 3e-2, "dx")
    _close(r.grad, rr.grad, 0.05, 3e-2, "dres")
    _close(nw.grad, nwr.grad, 0.5, 3e-2, "dnorm_w")
    _close(w.grad, wr.grad, 0.3, 3e-2, "dw")

    gu = _rand(T, 2 * I).requires_grad_()
    wd = _rand(H, I, scale=0.05).requires_grad_()
    y = ops.swiglu_linear(gu, wd)
    g = _rand(T, H)
    y.backward(g)
    gur, wdr = gu.detach().float().requires_grad_(), wd.detach().float().requires_grad_()
    a, b = gur.chunk(2, -1)
    yr = torch.nn.functional.linear(torch.nn.functional.silu(a) * b, wdr)
    yr.backward(g.float())
    _close(y, yr, 0.05, 2e-2, "swiglu_linear y")
    _close(gu.grad, gur.grad, 0.05, 3e-2, "dgate_up")
    _close(wd.grad, wdr.grad, 0.3, 3e-2, "dw_down")


def test_adamw_bf16_moments_close_to_fp32():
    cu = _cu()
    n = 50_000
    p0 = torch.randn(n, device=DEV)
    ma, m32, v32 = p0.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    mb, m16, v16 = p0.clone(), torch.zeros(n, device=DEV, dtype=torch.bfloat16), torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    pa, pb = p0.bfloat16(), p0.bfloat16()
    for step in range(1, 6):
        g = torch.randn(n, device=DEV).bfloat16()
        cu.adamw_step_(g, ma, m32, v32, pa, 1e-3, 0.9, 0.95, 1e-8, 0.1, step)
        cu.adamw_step_(g, mb, m16, v16, pb, 1e-3, 0.9, 0.95, 1e-8, 0.1, step)
    torch.testing.assert_close(ma, mb, atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("rows,cols", [(3000, 1152), (28672, 4304), (7, 8), (257, 264)])
def test_bias_colsum(rows, cols):
    cu = _cu()
    x = _rand(rows, cols)
    torch.testing.assert_close(cu._C.colsum(x), x.float().sum(0), atol=2e-2, rtol=1e-3)
    wide = _rand(rows, cols + 16)
    view = wide[:, 8:8 + cols]                    # a column slice: row stride larger than the width
    if view.data_ptr() % 16 == 0:
        torch.testing.assert_close(cu._colsum(view), view.float().sum(0), atol=2e-2, rtol=1e-3)


def test_layer_norm_linear_and_gelu_linear_match_unfused():
    T, H, N = 500, 1152, 4304
    x = _rand(T, H).requires_grad_()
    lw, lb = _rand(H, scale=0.5).requires_grad_(), _rand(H, scale=0.5).requires_grad_()
    w, b = _rand(N, H, scale=0.03).requires_grad_(), _rand(N, scale=0.1).requires_grad_()
    w2, b2 = _rand(H, N, scale=0.03).requires_grad_(), _rand(H, scale=0.1).requires_grad_()
    pre = ops.layer_norm_linear(x, lw, lb, w, b, 1e-6)
    y = ops.gelu_linear(pre, w2, b2, "tanh")
    g = _rand(T, H)
    y.backward(g)
    xr, lwr, lbr, wr, br, w2r, b2r = (t.detach().float().requires_grad_() for t in (x, lw, lb, w, b, w2, b2))
    pr = torch.nn.functional.linear(torch.nn.functional.layer_norm(xr, (H,), lwr, lbr, 1e-6), wr, br)
    yr = torch.nn.functional.linear(torch.nn.functional.gelu(pr, approximate="tanh"), w2r, b2r)
    yr.backward(g.float())
    _close(pre, pr, 0.05, 2e-2, "pre")
    _close(y, yr, 0.06, 3e-2, "y")
    _close(x.grad, xr.grad, 0.06, 4e-2, "dx")
    _close(w.grad, wr.grad, 0.4, 4e-2, "dw1")
    _close(w2.grad, w2r.grad, 0.8, 4e-2, "dw2")
    _close(b.grad, br.grad, 0.5, 4e-2, "db1")
    _close(b2.grad, b2r.grad, 0.5, 4e-2, "db2")
    _close(lw.grad, lwr.grad, 1.0, 4e-2, "dln_w")
    _close(lb.grad, lbr.grad, 1.0, 4e-2, "dln_b")


@pytest.mark.parametrize("T,H,I,E,k", [(300, 256, 128, 8, 2), (1000, 512, 256, 16, 4), (40, 128, 64, 8, 2)])
def test_moe_experts_grouped_gemm(T, H, I, E, k):
    """All experts in one grouped-GEMM launch per projection (some experts get no tokens) against the per-expert
    fp32 statement: outputs and the gradients of tokens, routing weights and both expert weight tensors."""
    cu = _cu()
    torch.manual_seed(0)
    x = _rand(T, H).requires_grad_()
    gate_up = _rand(E, 2 * I, H, scale=0.05).requires_grad_()
    down = _rand(E, H, I, scale=0.05).requires_grad_()
    logits = torch.randn(T, E, device=DEV)
    logits[:, E - 2:] = -1e9                      # the last two experts stay empty
    w, idx = ops.moe_router(logits, k, True)
    w = w.detach().to(torch.bfloat16).requires_grad_()
    out = ops.moe_experts(x, gate_up, down, w, idx)
    g = _rand(T, H)
    out.backward(g)
    cu.check_status()
    xr, gur, dr, wr = (t.detach().float().requires_grad_() for t in (x, gate_up, down, w))
    out_r = ref.moe_experts(xr, gur, dr, wr, idx)
    out_r.backward(g.float())
    _close(out, out_r, 0.03, 3e-2, "out")
    _close(x.grad, xr.grad, 0.03, 3e-2, "dx")
    _close(w.grad, wr.grad, 0.5, 5e-2, "dw_routing")   # a dot product of two bf16 rows of H elements
    _close(gate_up.grad, gur.grad, 0.3, 5e-2, "dgate_up")   # bf16 products summed over an expert's rows
    _close(down.grad, dr.grad, 0.3, 5e-2, "ddown")
    assert float(gate_up.grad[E - 1].abs().max()) == 0.0 and float(down.grad[E - 2].abs().max()) == 0.0


@pytest.mark.parametrize("T,E,k,renorm,dtype", [(777, 256, 8, True, torch.float32), (300, 256, 8, False, torch.bfloat16),
                                                 (64, 8, 2, True, torch.bfloat16), (1000, 100, 4, True, torch.float32)])
def test_moe_router_kernel(T, E, k, renorm, dtype):
    """softmax -> top-k -> renormalise in one kernel against the tensor-operation statement, forward and backward."""
    _cu()
    torch.manual_seed(1)
    logits = (torch.randn(T, E, device=DEV) * 2).to(dtype).requires_grad_()
    w, idx = ops.moe_router(logits, k, renorm)
    lr = logits.detach().float().requires_grad_()
    wr, idxr = ref.moe_router(lr, k, renorm)
    assert idx.dtype == torch.int64 and w.dtype == torch.float32
    # the same experts (as sets: equal probabilities may be ordered differently) with the same weights
    assert torch.equal(idx.sort(-1).values, idxr.sort(-1).values)
    _close(w.gather(1, idx.argsort(-1)), wr.gather(1, idxr.argsort(-1)), 1e-5, 1e-4, "weights")
    g = torch.randn(T, k, device=DEV)
    (w.gather(1, idx.argsort(-1)) * g).sum().backward()
    (wr.gather(1, idxr.argsort(-1)) * g).sum().backward()
    _close(logits.grad, lr.grad, 2e-3 if dtype == torch.bfloat16 else 1e-5, 2e-2 if dtype == torch.bfloat16 else 1e-3, "dlogits")


def test_moe_plan_is_a_stable_sort_by_expert():
    """Every slot gets the row that a stable sort by expert gives it inside its expert's 128-row tiles; rows that hold no
    slot are marked -1; run twice: identical placement."""
    cu = _cu()
    torch.manual_seed(2)
    T, k, E = 5000, 8, 256
    experts = torch.randint(0, E, (T, k), device=DEV)
    experts[experts == 7] = 8                                   # one empty expert
    from vlm_training_b200.ops.moe_cuda import MoePlan

    a, b = MoePlan(experts, E, k), MoePlan(experts, E, k)
    assert torch.equal(a.dest, b.dest) and torch.equal(a.slot_of_row, b.slot_of_row)
    flat = experts.reshape(-1)
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(a.counts.long(), counts)
    tiles = (counts + 127) // 128
    prefix = torch.cat((tiles.new_zeros(1), tiles.cumsum(0)))
    assert torch.equal(a.prefix.long(), prefix)
    order = torch.argsort(flat, stable=True)
    start = counts.cumsum(0) - counts
    e_sorted = flat[order]
    want = torch.empty_like(flat)
    want[order] = prefix[:-1][e_sorted] * 128 + (torch.arange(flat.numel(), device=DEV) - start[e_sorted])
    assert torch.equal(a.dest.long(), want)
    rows = a.slot_of_row.long()
    assert torch.equal(rows[want], torch.arange(flat.numel(), device=DEV)) and int((rows >= 0).sum()) == flat.numel()
    cu.check_status()


@pytest.mark.parametrize("reverse,head_major", [(False, False), (True, False), (False, True), (True, True)])
def test_gdn_scan_kernel_matches_loop(reverse, head_major):
    """The tcgen05 scan kernel against the same recurrence as a loop of fp32 tensor operations on the same bf16 inputs."""
    import numpy as np

    from vlm_training_b200.ops.gdn_scan import scan_torch

    cu = _cu()
    torch.manual_seed(5)
    H = 3
    count = np.array([1, 4, 2, 7], dtype=np.int32)
    first = np.concatenate(([0], np.cumsum(count)))[:-1].astype(np.int32)
    N = int(count.sum())
    x1, x2 = _rand(N, H, 64, 128, scale=0.06), _rand(N, H, 64, 128, scale=0.06)
    e = _rand(N, H, 64, 128, scale=0.5)
    decay = torch.rand(N, H, device=DEV) * 0.5 + 0.5
    ext = _rand(N, H, 128, 128, scale=0.2) if reverse else None
    ranges = (first, count, torch.from_numpy(np.stack((first, count), 1).copy()).to(DEV))
    if head_major:   # the same data in [H, N, ...] order
        x1, x2, e, decay = (t.transpose(0, 1).contiguous() for t in (x1, x2, e, decay))
        ext = ext.transpose(0, 1).contiguous() if ext is not None else None
    y, states = cu.gdn_scan(x1, x2, e, decay, ext, ranges, reverse, head_major)
    torch.cuda.synchronize()
    cu.check_status()
    assert y.dtype == torch.bfloat16 and states.dtype == torch.bfloat16
    y_ref, s_ref = scan_torch(x1, x2, e, decay, ext, first, count, reverse, head_major)
    _close(y, y_ref, atol=0.03, rtol=3e-2, what="scan Y")
    _close(states, s_ref, atol=0.03, rtol=3e-2, what="scan states")
    y2, states2 = cu.gdn_scan(x1, x2, e, decay, ext, ranges, reverse, head_major)       # no atomics: bit-reproducible
    assert torch.equal(y, y2) and torch.equal(states, states2)


@pytest.mark.parametrize("native_chunks", [True, False])
def test_gated_delta_rule_scan_path_matches_reference(native_chunks, monkeypatch):
    """Head size 128 takes the scan-kernel path, with the work inside the chunks as tcgen05 kernels too or as tensor
    operations; outputs and all five gradients against the fp32 reference."""
    from vlm_training_b200.ops import gdn_scan

    monkeypatch.setenv("VLMT_GDN_CHUNK", "1" if native_chunks else "0")
    calls0 = dict(gdn_scan.NATIVE_CALLS)
    torch.manual_seed(11)
    T, H, D = 700, 2, 128
    cu_list = [0, 130, 130, 200, 641, 700]
    cu_t = torch.tensor(cu_list, device=DEV, dtype=torch.int32)

    def mk():
        q, k, v = _rand(T, H, D), _rand(T, H, D), _rand(T, H, D)
        g = (-torch.rand(T, H, device=DEV) * 0.3).float()
        b = torch.rand(T, H, device=DEV).to(torch.bfloat16)
        return [t.requires_grad_() for t in (q, k, v, g, b)]

    ins = mk()
    go = _rand(T, H, D, scale=0.5)
    ins_ref = [t.detach().float().requires_grad_() for t in ins]
    want = ref.gated_delta_rule(*ins_ref, cu_t)
    want.backward(go.float())
    got = ops.gated_delta_rule(*ins, cu_t, None, 64, cu_host=cu_list)
    got.backward(go)
    _cu().check_status()
    _close(got, want, atol=0.03, rtol=4e-2, what="gdn out")
    for name, a, b in zip("qkvgb", ins, ins_ref):
        scale = float(b.grad.abs().max())
        _close(a.grad, b.grad, atol=0.03 * scale + 1e-3, rtol=6e-2, what=f"gdn d{name}")
    ran = gdn_scan.NATIVE_CALLS["forward"] - calls0["forward"], gdn_scan.NATIVE_CALLS["backward"] - calls0["backward"]
    assert ran == ((1, 1) if native_chunks else (0, 0))


@pytest.mark.parametrize("cu_list,H", [([0, 64, 128, 129, 512], 4), ([0, 1, 3, 1000], 3), ([0, 2048], 8), ([0, 300, 300, 900], 2)])
def test_gated_delta_rule_native_chunks_shapes(cu_list, H):
    """Chunk boundaries that coincide with document ends, documents of one token, a long document, rows that end before
    the tensor does (trailing tokens belong to no document) and strided q / k / v (slices of one projection)."""
    from vlm_training_b200.ops import gdn_scan

    torch.manual_seed(5)
    T, D = cu_list[-1] + (24 if len(cu_list) == 4 and H == 2 else 0), 128
    cu_t = torch.tensor(cu_list, device=DEV, dtype=torch.int32)
    proj = _rand(T, 3 * H * D).requires_grad_()
    g = (-torch.rand(T, H, device=DEV) * 0.2).float().requires_grad_()
    b = torch.rand(T, H, device=DEV).requires_grad_()
    proj_ref, g_ref, b_ref = (t.detach().float().requires_grad_() for t in (proj, g, b))

    def split(p):
        q, k, v = p.split(H * D, dim=-1)
        return q.reshape(T, H, D), k.reshape(T, H, D), v.reshape(T, H, D)

    calls0 = gdn_scan.NATIVE_CALLS["forward"]
    got = ops.gated_delta_rule(*split(proj), g, b, cu_t, None, 64, cu_host=cu_list)
    assert gdn_scan.NATIVE_CALLS["forward"] == calls0 + 1
    want = ref.gated_delta_rule(*split(proj_ref), g_ref, b_ref, cu_t)
    go = _rand(T, H, D, scale=0.5)
    got.backward(go)
    want.backward(go.float())
    _cu().check_status()
    Tc = cu_list[-1]
    _close(got[:Tc], want[:Tc], atol=0.03, rtol=4e-2, what="gdn out")
    assert Tc == T or float(got[Tc:].detach().abs().max()) == 0.0
    for name, a, r in (("proj", proj, proj_ref), ("g", g, g_ref), ("beta", b, b_ref)):
        scale = float(r.grad.abs().max())
        _close(a.grad, r.grad, atol=0.03 * scale + 1e-3, rtol=6e-2, what=f"gdn d{name}")
