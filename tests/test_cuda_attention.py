"""tcgen05 varlen attention against the fp32 per-document softmax(QK^T)V statement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from vlm_training_b200 import ops
from vlm_training_b200.ops import reference as ref

DEV = "cuda"


def _close(got, want, atol, rtol, what=""):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4g}, max ref {want.abs().max().item():.4g}, " \
                                     f"frac bad {(err > tol).float().mean().item():.4g}"


CASES = [
    # (doc lengths, Hq, Hkv, D, causal)
    ([128], 1, 1, 128, True),
    ([256], 2, 1, 128, True),
    ([100, 1, 300, 57], 4, 2, 128, True),
    ([513, 127, 129], 4, 1, 64, True),
    ([196, 196, 1024], 4, 4, 72, False),   # ViT: head_dim 72 runs in a 128-wide tile whose channels 72.. TMA zero-fills
    ([300, 90], 2, 1, 40, True),           # 64-wide tile, 24 channels zero-filled
    ([260, 513], 4, 2, 96, True),
    ([129, 700], 2, 2, 120, False),
    ([333], 2, 1, 100, True),              # not a multiple of 8: padded to 104 by a copy
    ([700], 8, 2, 128, False),
    ([1500, 260, 40], 2, 1, 128, True),
    ([900, 130], 2, 2, 64, False),
    ([128], 1, 1, 256, True),              # head size 256: the single-tile kernels (Qwen3.5 full-attention layers)
    ([300, 200], 4, 2, 256, True),
    ([700], 4, 1, 256, False),
    ([1500, 260, 40, 1, 65], 2, 1, 256, True),
    ([384, 640], 4, 4, 256, False),
    ([500], 2, 2, 192, True),              # padded to 256
]


@pytest.mark.parametrize("lens,Hq,Hkv,D,causal", CASES)
def test_attention_fwd_bwd(lens, Hq, Hkv, D, causal):
    from vlm_training_b200.ops import cuda as cu

    torch.manual_seed(0)
    T = sum(lens)
    cu_seq = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    q = (torch.randn(T, Hq, D, device=DEV)).bfloat16().requires_grad_()
    k = (torch.randn(T, Hkv, D, device=DEV)).bfloat16().requires_grad_()
    v = (torch.randn(T, Hkv, D, device=DEV)).bfloat16().requires_grad_()
    o = ops.attention_varlen(q, k, v, cu_seq, max(lens), causal, None)
    g = torch.randn(T, Hq, D, device=DEV).bfloat16()
    o.backward(g)
    cu.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_r = ref.attention_varlen(qr, kr, vr, cu_seq, max(lens), causal, None)
    o_r.backward(g.float())
    _close(o, o_r, 0.02, 2e-2, "out")
    _close(q.grad, qr.grad, 0.05, 3e-2, "dq")
    _close(k.grad, kr.grad, 0.05, 3e-2, "dk")
    _close(v.grad, vr.grad, 0.05, 3e-2, "dv")


@pytest.mark.parametrize("D", [128, 256])
def test_attention_is_repeatable(D):
    T, Hq, Hkv = 1000, 4, 2
    cu_seq = torch.tensor([0, 300, 1000], dtype=torch.int32, device=DEV)
    q, k, v = (torch.randn(T, h, D, device=DEV).bfloat16().requires_grad_() for h in (Hq, Hkv, Hkv))
    g = torch.randn(T, Hq, D, device=DEV).bfloat16()
    outs = []
    for _ in range(2):
        q.grad = k.grad = v.grad = None
        o = ops.attention_varlen(q, k, v, cu_seq, 700, True, None)
        o.backward(g)
        outs.append((o.detach().clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("D", [128, 256])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_growing_scores(causal, D):
    """Scores that keep growing along the keys make the running row max jump by far more than the lazy-rescale
    threshold several times per row, so the in-TMEM rescale of the output accumulator is exercised."""
    from vlm_training_b200.ops import cuda as cu

    torch.manual_seed(1)
    lens, Hq, Hkv = [1100, 300], 2, 1
    T = sum(lens)
    cu_seq = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ramp = torch.linspace(0.2, 6.0, T, device=DEV)[:, None, None]
    base = torch.randn(1, 1, D, device=DEV)
    q = (base + 0.3 * torch.randn(T, Hq, D, device=DEV)).bfloat16().requires_grad_()
    k = (ramp * (base + 0.3 * torch.randn(T, Hkv, D, device=DEV))).bfloat16().requires_grad_()
    v = torch.randn(T, Hkv, D, device=DEV).bfloat16().requires_grad_()
    o = ops.attention_varlen(q, k, v, cu_seq, max(lens), causal, None)
    g = torch.randn(T, Hq, D, device=DEV).bfloat16()
    o.backward(g)
    cu.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_r = ref.attention_varlen(qr, kr, vr, cu_seq, max(lens), causal, None)
    o_r.backward(g.float())
    _close(o, o_r, 0.03, 3e-2, "out")
    _close(q.grad, qr.grad, 0.08, 5e-2, "dq")
    _close(k.grad, kr.grad, 0.08, 5e-2, "dk")
    _close(v.grad, vr.grad, 0.08, 5e-2, "dv")


def test_attention_reads_strided_heads_in_place():
    """q, k, v as slices of one fused projection ``[T, 3, H, 72]`` (the ViT layout): read through strided tensor maps,
    no padded or contiguous copies; gradients come back through the slices."""
    from vlm_training_b200.ops import cuda as cu

    torch.manual_seed(3)
    lens, H, D = [196, 1024, 77], 4, 72
    T = sum(lens)
    cu_seq = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    qkv = torch.randn(T, 3 * H * D, device=DEV).bfloat16().requires_grad_()
    q, k, v = qkv.view(T, 3, H, D).unbind(1)
    assert not v.is_contiguous()
    o = ops.attention_varlen(q, k, v, cu_seq, max(lens), False, None)
    g = torch.randn(T, H, D, device=DEV).bfloat16()
    o.backward(g)
    cu.check_status()
    ref_in = qkv.detach().float().requires_grad_()
    qr, kr, vr = ref_in.view(T, 3, H, D).unbind(1)
    o_r = ref.attention_varlen(qr, kr, vr, cu_seq, max(lens), False, None)
    o_r.backward(g.float())
    _close(o, o_r, 0.02, 2e-2, "out")
    _close(qkv.grad, ref_in.grad, 0.05, 3e-2, "dqkv")


@pytest.mark.parametrize("L,b0,B,kk", [(3000, 1024, 1024, 512), (700, 0, 700, 64), (5000, 4096, 904, 2048), (300, 256, 44, 128)])
def test_dsa_indexer_scores_and_topk(L, b0, B, kk):
    """Indexer scores on the tensor cores + radix-select top-k against fp32 scores and torch.topk: the selected sets are
    compared through their scores (ties may be broken differently), indices must be causal and distinct."""
    from vlm_training_b200.ops import cuda as cu

    torch.manual_seed(4)
    pre = 37                                     # the document starts in the middle of the packed row
    T = pre + L + 11
    iq = (torch.randn(T, 4, 64, device="cuda") * 0.3).bfloat16()
    ik = (torch.randn(T, 64, device="cuda") * 0.3).bfloat16()
    w = torch.randn(T, 4, device="cuda")
    sel = cu._C.dsa_select(iq, ik, w, pre + b0, b0, pre, B, min(kk, b0 + B))
    cu.check_status()
    kq = min(kk, b0 + B)
    assert sel.shape == (B, kq)
    sc = torch.einsum("thd,sd->ths", iq[pre + b0:pre + b0 + B].float(), ik[pre:pre + b0 + B].float()).relu()
    sc = (sc * w[pre + b0:pre + b0 + B].unsqueeze(-1)).sum(1)
    qpos = torch.arange(b0, b0 + B, device="cuda").unsqueeze(1)
    kpos = torch.arange(b0 + B, device="cuda").unsqueeze(0)
    sc = sc.masked_fill(kpos > qpos, float("-inf"))
    want = sc.topk(kq, dim=-1).values                                    # [B, kq], descending, -inf where fewer causal keys
    valid = sel >= 0
    assert bool(((sel <= qpos) | ~valid).all()), "a selected key lies after its query"
    n_causal = (qpos.squeeze(1) + 1).clamp(max=kq)
    assert torch.equal(valid.sum(1), n_causal)
    srt = torch.where(valid, sel, torch.full_like(sel, -1)).sort(dim=1).values
    dup = (srt[:, 1:] == srt[:, :-1]) & (srt[:, 1:] >= 0)
    assert not bool(dup.any()), "an index was selected twice"
    got = torch.where(valid, sc.gather(1, sel.clamp(min=0).long()), torch.full_like(want, float("-inf"))).sort(dim=1, descending=True).values
    finite = torch.isfinite(want)
    assert torch.equal(finite, torch.isfinite(got))
    torch.testing.assert_close(got[finite], want[finite], atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("D,Hkv,rep,L,B,kk", [(256, 2, 8, 700, 96, 300), (256, 1, 8, 3000, 40, 2048), (64, 2, 2, 300, 50, 64), (128, 1, 4, 513, 33, 2048)])
def test_dsa_selected_attention_kernels(D, Hkv, rep, L, B, kk):
    """Selected-key attention kernels (forward and backward) against the gathered dense softmax in float32."""
    from vlm_training_b200.ops import dsa_cuda

    torch.manual_seed(2)
    kk = min(kk, L)
    q = (torch.randn(B, Hkv * rep, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    k = (torch.randn(L, Hkv, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    v = torch.randn(L, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    sel = torch.stack([torch.randperm(L, device="cuda")[:kk] for _ in range(B)])
    valid = torch.rand(B, kk, device="cuda") > 0.3
    valid[:, 0] = True
    valid[1] = False                       # a query without any key: zero output, zero gradients
    scale = D ** -0.5
    go = torch.randn(B, Hkv * rep, D, device="cuda").to(torch.bfloat16)
    sel32 = torch.where(valid, sel, -1).to(torch.int32)
    got = dsa_cuda._SelectedAttention.apply(q, k, v, sel32, scale)
    got.backward(go)
    grads = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    v2 = valid.clone()
    v2[1, 0] = True                        # the tensor form cannot softmax an empty row; row 1 is compared separately
    want = dsa_cuda._block_attention(q, k, v, sel, v2, scale, rep)
    mask = torch.ones(B, 1, 1, device="cuda")
    mask[1] = 0
    (want * mask).backward(go.float())
    assert float(got[1].detach().abs().max()) == 0.0
    torch.testing.assert_close(got.float() * mask, want * mask, atol=2e-2, rtol=2e-2)
    for name, a, t in zip("qkv", grads, (q, k, v)):
        ref = t.grad.float()
        tol = 2e-2 * float(ref.abs().max()) + 1e-3
        assert float((a.float() - ref).abs().max()) <= tol, (name, float((a.float() - ref).abs().max()), tol)
    a2 = dsa_cuda._SelectedAttention.apply(q, k, v, sel32, scale)
    assert torch.equal(a2, got)
