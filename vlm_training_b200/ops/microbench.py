"""Per-kernel micro-benchmarks (CUDA-event timing, L2 flushed between iterations) and roofline fractions.

    python -m vlm_training_b200.ops.microbench gemm --m 8192 --n 6144 --k 4096 [--layout fwd|dgrad|wgrad]
    python -m vlm_training_b200.ops.microbench attention --tokens 8192 --docs 1 [--backward]
    python -m vlm_training_b200.ops.microbench rmsnorm | swiglu | qkv_rope | ce | adamw | moe | fused_adamw | gemm_ag
    python -m vlm_training_b200.ops.microbench gdn_scan --tokens 16384 --docs 1 [--backward]   |   conv1d [--backward]   |   dsa [--backward]
    python -m vlm_training_b200.ops.microbench all            # the table used in the roofline report

Each line is JSON: algorithmic FLOPs / bytes, median milliseconds, achieved rate, and the fraction of the
measured peak (``MEASURED_PEAKS.json`` in the working directory when present: burst cuBLAS bf16 rate and
STREAM-style copy bandwidth; otherwise 1.59 PFLOP/s and 6.65 TB/s).  ``--iters 1 --warmup 0 --no-flush`` gives
a run small enough to put under a profiler.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def peaks() -> dict:
    for path in (os.environ.get("VLMT_MEASURED_PEAKS", ""), "MEASURED_PEAKS.json"):
        if path and os.path.exists(path):
            with open(path) as fh:
                d = json.load(fh)
            return {"tflops": float(d["bf16_tflops"]), "gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "gbs": 6650.0, "source": "fallback"}


class Timer:
    def __init__(self, iters: int, warmup: int, flush: bool):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2]


def _report(name, shape, ms, flops=None, nbytes=None):
    pk = peaks()
    out = {"kernel": name, "shape": shape, "ms": round(ms, 4)}
    if flops is not None:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_" + pk["source"] + "_gemm_peak"] = round(flops / ms / 1e9 / pk["tflops"], 3)
    if nbytes is not None:
        out["gbs"] = round(nbytes / ms / 1e6, 1)
        out["frac_of_" + pk["source"] + "_copy_bw"] = round(nbytes / ms / 1e6 / pk["gbs"], 3)
    print(json.dumps(out), flush=True)
    return out


def _r(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def bench_gemm(t: Timer, m, n, k, layout="fwd"):
    from . import cuda as cu

    if layout == "fwd":
        a, b = _r(m, k), _r(n, k)
        fn = lambda: cu._gemm(a, b)
    elif layout == "dgrad":  # dX[m,n] = dY[m,k] W[k,n]
        a, b = _r(m, k), _r(k, n)
        fn = lambda: cu._gemm(a, b, b_mn=True)
    elif layout == "wgrad_acc":  # the product is added into an existing gradient (TMA reduce-add; split over K where that fills the SMs)
        a, b = _r(k, m), _r(k, n)
        out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
        fn = lambda: cu._gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
    else:  # wgrad: dW[m,n] = dY[k,m]^T X[k,n]
        a, b = _r(k, m), _r(k, n)
        fn = lambda: cu._gemm(a, b, a_mn=True, b_mn=True)
    return _report(f"gemm_{layout}", [m, n, k], t(fn), flops=2.0 * m * n * k)


def bench_attention(t: Timer, tokens, docs, hq=32, hkv=8, d=128, causal=True, backward=False, library=False):
    """``library``: time torch's varlen attention (the reference's kernel) on the same inputs instead of ours."""
    from .. import ops

    lens = [tokens // docs] * docs
    cu_seq = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q, k, v = (_r(tokens, h, d).requires_grad_() for h in (hq, hkv, hkv))
    g = _r(tokens, hq, d)
    fl = sum(4.0 * L * L * d * hq * (0.5 if causal else 1.0) for L in lens)
    if library:
        from torch.nn.attention.varlen import varlen_attn

        fn = lambda: varlen_attn(q, k, v, cu_seq, cu_seq, max(lens), max(lens), window_size=(-1, 0) if causal else (-1, -1))
        tag = "library_varlen_attn"
    else:
        fn = lambda: ops.attention_varlen(q, k, v, cu_seq, max(lens), causal, None)
        tag = "attention"
    if not backward:
        with torch.no_grad():
            ms = t(fn)
        return _report(tag + "_fwd", [tokens, docs, hq, hkv, d, int(causal)], ms, flops=fl)

    def fb():
        fn().backward(g)
    return _report(tag + "_fwd_bwd", [tokens, docs, hq, hkv, d, int(causal)], t(fb), flops=3.5 * fl)


def bench_rmsnorm(t: Timer, rows=8192, dim=4096):
    from . import cuda as cu

    x, w = _r(rows, dim), _r(dim)
    ms = t(lambda: cu._C.rmsnorm_fwd(x, None, w, 1e-6, False))
    _report("rmsnorm_fwd", [rows, dim], ms, nbytes=2.0 * rows * dim * 2)
    y, rstd = cu._C.rmsnorm_fwd(x, None, w, 1e-6, False)
    ms = t(lambda: cu._C.rmsnorm_bwd(y, x, w, rstd, None, False))
    return _report("rmsnorm_bwd", [rows, dim], ms, nbytes=3.0 * rows * dim * 2)


def bench_layernorm(t: Timer, rows=28672, dim=1152):
    from . import cuda as cu

    x, w, b = _r(rows, dim), _r(dim), _r(dim)
    ms = t(lambda: cu._C.layernorm_fwd(x, w, b, 1e-6))
    _report("layernorm_fwd", [rows, dim], ms, nbytes=2.0 * rows * dim * 2)
    y, mean, rstd = cu._C.layernorm_fwd(x, w, b, 1e-6)
    ms = t(lambda: cu._C.layernorm_bwd(y, x, w, mean, rstd))
    return _report("layernorm_bwd", [rows, dim], ms, nbytes=3.0 * rows * dim * 2)


def bench_rope_vision(t: Timer, tokens=28672, heads=16, d=72):
    """The ViT's rotary embedding on the q slice of a fused qkv projection (strided input, contiguous output)."""
    from . import cuda as cu

    qkv = _r(tokens, 3 * heads * d)
    q = qkv[:, : heads * d].view(tokens, heads, d)
    ang = torch.rand(tokens, d, device="cuda") * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    ms = t(lambda: cu._C.rope_generic(q, cos, sin, False, d))
    return _report("rope_vision_fwd", [tokens, heads, d], ms, nbytes=2.0 * tokens * heads * d * 2)


def bench_gelu(t: Timer, rows=28672, dim=4304):
    from . import cuda as cu

    x, dy = _r(rows, dim), _r(rows, dim)
    ms = t(lambda: cu._C.gelu_fwd(x, True))
    _report("gelu_tanh_fwd", [rows, dim], ms, nbytes=2.0 * rows * dim * 2)
    ms = t(lambda: cu._C.gelu_bwd(dy, x, True))
    return _report("gelu_tanh_bwd", [rows, dim], ms, nbytes=3.0 * rows * dim * 2)


def bench_swiglu(t: Timer, rows=8192, inter=12288):
    from . import cuda as cu

    gu = _r(rows, 2 * inter)
    ms = t(lambda: cu._C.swiglu_fwd(gu))
    _report("swiglu_fwd", [rows, inter], ms, nbytes=3.0 * rows * inter * 2)
    d = _r(rows, inter)
    ms = t(lambda: cu._C.swiglu_bwd(d, gu))
    return _report("swiglu_bwd", [rows, inter], ms, nbytes=5.0 * rows * inter * 2)


def bench_qkv_rope(t: Timer, tokens=8192, hq=32, hkv=8, d=128):
    from . import cuda as cu

    qkv = _r(tokens, (hq + 2 * hkv) * d)
    w = _r(d)
    ang = torch.rand(tokens, d // 2, device="cuda")
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos().contiguous(), emb.sin().contiguous()
    ms = t(lambda: cu._C.qkv_norm_rope_fwd(qkv, hq, hkv, d, w, w, cos, sin, 1e-6, False, False))
    return _report("qkv_norm_rope_fwd", [tokens, hq, hkv, d], ms, nbytes=2.0 * qkv.numel() * 2)


def bench_ce(t: Timer, tokens=4096, hidden=4096, vocab=151936):
    from . import cuda as cu

    logits = _r(tokens, vocab)
    tgt = torch.randint(0, vocab, (tokens,), device="cuda")
    ms = t(lambda: cu._C.ce_fwd_bwd_(logits, tgt, 1.0, -100))
    return _report("ce_softmax_grad", [tokens, vocab], ms, nbytes=2.0 * tokens * vocab * 2)


def bench_adamw(t: Timer, n=1 << 28):
    from . import cuda as cu

    g = torch.randn(n, device="cuda").bfloat16()
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    master, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    ms = t(lambda: cu._C.adamw_(g, master, m, v, p, 1e-4, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, False))
    return _report("adamw_fp32_state", [n], ms, nbytes=n * (2 + 12 + 12 + 2.0))


def bench_moe(t: Timer, tokens=16384, hidden=2048, inter=512, experts=256, topk=8):
    """Routed experts of one MoE layer (grouped GEMMs, forward + backward) with a random router."""
    from .. import ops

    x = _r(tokens, hidden).requires_grad_()
    gate_up = _r(experts, 2 * inter, hidden, scale=0.02).requires_grad_()
    down = _r(experts, hidden, inter, scale=0.02).requires_grad_()
    w, idx = ops.moe_router(torch.randn(tokens, experts, device="cuda"), topk, True)
    w = w.to(torch.bfloat16)
    g = _r(tokens, hidden)

    def fb():
        ops.moe_experts(x, gate_up, down, w, idx).backward(g)
    flops = 3.0 * tokens * topk * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden)
    return _report("moe_experts_fwd_bwd", [tokens, hidden, inter, experts, topk], t(fb), flops=flops)


def bench_gdn_scan(t: Timer, tokens=16384, docs=1, heads=32, reverse=False):
    """The chunk-to-chunk scan of the gated delta rule: ``tokens / 64`` chunks split evenly over ``docs`` documents."""
    import numpy as np

    from . import cuda as cu

    n = tokens // 64
    per = n // docs
    first = (np.arange(docs) * per).astype(np.int32)
    count = np.full(docs, per, dtype=np.int32)
    ranges = (first, count, torch.from_numpy(np.stack((first, count), 1).copy()).cuda())
    x1, x2 = _r(n, heads, 64, 128, scale=0.05), _r(n, heads, 64, 128, scale=0.05)
    e = _r(n, heads, 64, 128, scale=0.5)
    decay = torch.rand(n, heads, device="cuda") * 0.3 + 0.7
    ext = _r(n, heads, 128, 128, scale=0.1) if reverse else None
    ms = t(lambda: cu.gdn_scan(x1, x2, e, decay, ext, ranges, reverse, False))
    nbytes = 2.0 * n * heads * (4 * 64 * 128 + (2 if reverse else 1) * 128 * 128)   # 3 operand tiles in, Y and states out (+ ext in)
    out = _report("gdn_scan_bwd" if reverse else "gdn_scan_fwd", [tokens, docs, heads], ms, nbytes=nbytes)
    print(json.dumps({"kernel": "gdn_scan", "us_per_chunk_step": round(ms * 1e3 / per, 3)}))
    return out


def bench_gdn(t: Timer, tokens=16384, docs=16, heads=32, backward=False):
    """The whole gated delta rule (prepare -> scan -> output, and back) on one packed row; ``VLMT_GDN_CHUNK=0`` times the
    form with tensor operations inside the chunks.  The byte count is the op's inputs and outputs once (q, k, v, o and, with
    the backward pass, their gradients), so the fraction says how far the op is from a pass over its own tensors."""
    from .. import ops

    per = tokens // docs
    cu_list = [i * per for i in range(docs)] + [tokens]
    cu_t = torch.tensor(cu_list, device="cuda", dtype=torch.int32)
    q, k, v = (_r(tokens, heads, 128, scale=0.5).requires_grad_() for _ in range(3))
    g = (-torch.rand(tokens, heads, device="cuda") * 0.2).requires_grad_()
    b = torch.rand(tokens, heads, device="cuda").requires_grad_()
    go = _r(tokens, heads, 128, scale=0.5)
    io = 4.0 * tokens * heads * 128 * 2
    if not backward:
        with torch.no_grad():
            ms = t(lambda: ops.gated_delta_rule(q, k, v, g, b, cu_t, None, 64, cu_host=cu_list))
        return _report("gated_delta_rule_fwd", [tokens, docs, heads], ms, nbytes=io)

    def fb():
        o = ops.gated_delta_rule(q, k, v, g, b, cu_t, None, 64, cu_host=cu_list)
        torch.autograd.grad(o, (q, k, v, g, b), go)
    return _report("gated_delta_rule_fwd_bwd", [tokens, docs, heads], t(fb), nbytes=2.0 * io)


def bench_gemm_wgather(t: Timer, m=8192, n=6144, k=4096, world=2):
    """The parameter all-gather -> GEMM kernel run as rank 0 of ``world`` on one GPU: the peers' shards are staged in local
    memory, so no link is crossed; shows what the copy warps and the gated B tiles cost next to the plain GEMM."""
    from . import cuda as cu

    shard = (n * k // world + 4096) // 8 * 8
    flat = _r(shard * world, scale=0.05)
    shards = [flat[r * shard:(r + 1) * shard].clone() for r in range(world)]
    bucket = torch.zeros_like(flat)
    w = bucket[1024:1024 + n * k].view(n, k)
    x = _r(m, k)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    sync = torch.zeros(2 * world, dtype=torch.int32, device="cuda")
    ptrs = [s_.data_ptr() for s_ in shards]
    epoch = [0]

    def fn():
        epoch[0] += 1
        cu._C.gemm_wgather(x, w, out, None, bucket, ptrs, shard, 0, sync, epoch[0])
    _report(f"gemm_weight_gather_rank0_of_{world}", [m, n, k], t(fn), flops=2.0 * m * n * k)
    return _report("gemm_fwd_same_shape", [m, n, k], t(lambda: cu._gemm(x, w)), flops=2.0 * m * n * k)


def bench_conv1d(t: Timer, tokens=16384, channels=8192, backward=False):
    from .. import ops
    from . import reference as ref

    x = _r(tokens, channels).requires_grad_()
    w = _r(channels, 4, scale=0.5).requires_grad_()
    cu_seq = torch.tensor([0, tokens // 3, tokens], device="cuda", dtype=torch.int32)
    seq_idx = ref.seq_idx_from_cu(cu_seq, tokens)
    g = _r(tokens, channels)
    if backward:
        y = ops.causal_conv1d_silu(x, w, seq_idx)
        ms = t(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True))
        return _report("conv1d_silu_bwd", [tokens, channels], ms, nbytes=2.0 * tokens * channels * 3)
    with torch.no_grad():
        ms = t(lambda: ops.causal_conv1d_silu(x, w, seq_idx))
    return _report("conv1d_silu_fwd", [tokens, channels], ms, nbytes=2.0 * tokens * channels * 2)


def bench_dsa(t: Timer, queries=1024, keys=16384, topk=2048, hkv=2, rep=8, d=256, backward=False):
    """Selected-key attention of one query block: every query reads its own ``topk`` rows of a ``keys``-row document."""
    from . import dsa_cuda

    q = _r(queries, hkv * rep, d, scale=0.5).requires_grad_()
    k = _r(keys, hkv, d, scale=0.5).requires_grad_()
    v = _r(keys, hkv, d).requires_grad_()
    sel = torch.rand(queries, keys, device="cuda").topk(topk, dim=-1).indices.to(torch.int32)
    g = _r(queries, hkv * rep, d)
    gathered = 2.0 * queries * hkv * topk * d * 2     # key and value rows read by the forward pass
    if backward:
        o = dsa_cuda._SelectedAttention.apply(q, k, v, sel, d ** -0.5)
        ms = t(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True))
        return _report("dsa_selected_attention_bwd", [queries, keys, topk, hkv, rep, d], ms, nbytes=2.0 * gathered)
    with torch.no_grad():
        ms = t(lambda: dsa_cuda._SelectedAttention.apply(q, k, v, sel, d ** -0.5))
    return _report("dsa_selected_attention_fwd", [queries, keys, topk, hkv, rep, d], ms, nbytes=gathered)


def bench_fused_adamw(t: Timer, n=1 << 27, state=torch.float32):
    """The reduce-scatter + AdamW + all-gather kernel on a domain of one rank (no peers): what it costs when only the
    memory system limits it; the multi-rank timings are in ``parallel.microbench_comm``."""
    from . import cuda as cu

    g = _r(n)
    p = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    master = torch.zeros(n, device="cuda")
    m, v = torch.zeros(n, device="cuda", dtype=state), torch.zeros(n, device="cuda", dtype=state)
    fn = lambda: cu._C.fused_rs_adamw_ag([g.data_ptr()], [p.data_ptr()], 0, 0, 1, 0, n, master, m, v, 0, 1e-5, 0.9, 0.999, 1e-8, 0.01,
                                         0.1, 0.001, 1.0, True)
    sb = 4 if state == torch.float32 else 2
    nbytes = n * (2 + 2 + 4 + 2 * sb) + n * (4 + 2 * sb + 2)   # grad read + cleared, state read, state + parameter written
    return _report(f"fused_rs_adamw_ag_one_rank_{'fp32' if sb == 4 else 'bf16'}_moments", [n], t(fn), nbytes=nbytes)


def bench_gemm_ag(t: Timer, m=8192, n=3072, k=4096, b_mn=False):
    """The all-gather -> GEMM kernel run as rank 0 of two on one GPU: the peer's rows are already in the gathered buffer
    and its flag is set, the kernel's own push goes into a second local buffer.  Shows the cost of the push warps and the
    two-source A operand next to the plain GEMM of the same shape (no link is crossed here)."""
    from . import cuda as cu

    R = m // 2
    x_loc, x_full, peer_buf = _r(R, k), _r(m, k), _r(m, k)
    w = _r(k, n) if b_mn else _r(n, k)
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    peer_flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[1] = 1 << 30
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    fn = lambda: cu._C.gemm_ag(x_loc, x_full, w, y, [x_full.data_ptr(), peer_buf.data_ptr()], [flags.data_ptr(), peer_flags.data_ptr()],
                               0, counter, 5, 0, b_mn)
    return _report("gemm_all_gather_rank0_of_2_" + ("dgrad" if b_mn else "fwd"), [m, n, k], t(fn), flops=2.0 * m * n * k)


def bench_gemm_fp8(t: Timer, m=8192, n=6144, k=4096, accumulate=False):
    """The FP8 GEMM alone (operands already quantised) next to the bf16 GEMM of the same shape."""
    from . import cuda as cu

    a8, _, ra = cu._C.fp8_quantize(_r(m, k), 0, True, False)
    b8, _, rb = cu._C.fp8_quantize(_r(n, k), 0, True, False)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    fn = lambda: cu._C.gemm_fp8(a8, b8, out, ra, rb, 0, 0, accumulate)
    return _report("gemm_fp8" + ("_acc" if accumulate else ""), [m, n, k], t(fn), flops=2.0 * m * n * k)


def bench_linear_fp8(t: Timer, m=8192, n=6144, k=4096):
    """Forward + backward of one linear layer (three GEMMs) in FP8, quantisation kernels included, and in bf16."""
    from . import cuda as cu

    x = _r(m, k).requires_grad_(True)
    dy = _r(m, n)
    out = []
    for fp8 in (True, False):
        w = torch.nn.Parameter(_r(n, k))
        w._vlmt_fp8 = fp8

        def fn():
            x.grad = None
            w.grad = None
            cu.linear(x, w).backward(dy)

        out.append(_report("linear_fwd_bwd_" + ("fp8" if fp8 else "bf16"), [m, n, k], t(fn), flops=6.0 * m * n * k))
    nb = (m * k + n * k + m * n) * 2
    fnq = lambda: cu._C.fp8_quantize(x.detach(), 0, True, True)
    out.append(_report("fp8_quantize_both_layouts", [m, k], t(fnq), nbytes=m * k * (2 + 2 + 1 + 1)))
    return out


def bench_gemm_rs_push(t: Timer, m=8192, n=4096, k=6144, b_mn=False):
    """The GEMM -> reduce-scatter-push kernel run as rank 0 of two on one GPU: the epilogue stores the rows of each owner
    into that owner's staging block, both of which are local buffers here (no link is crossed), so the figure is the
    kernel's own cost next to the plain GEMM of the same shape."""
    from . import cuda as cu

    rows = m // 2
    x = _r(m, k)
    w = _r(k, n) if b_mn else _r(n, k)
    mine = torch.empty(2, rows, n, dtype=torch.bfloat16, device="cuda")
    peer = torch.empty(2, rows, n, dtype=torch.bfloat16, device="cuda")
    fn = lambda: cu._C.gemm_rs_push(x, w, [mine.data_ptr(), peer.data_ptr()], rows, b_mn)
    return _report("gemm_rs_push_rank0_of_2_" + ("dgrad" if b_mn else "fwd"), [m, n, k], t(fn), flops=2.0 * m * n * k)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attention", "rmsnorm", "layernorm", "rope_vision", "gelu", "swiglu", "qkv_rope", "ce", "adamw", "moe", "gdn_scan", "gdn", "conv1d", "dsa", "fused_adamw", "gemm_ag", "gemm_rs_push", "gemm_wgather", "gemm_fp8", "linear_fp8", "all"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="fwd", choices=["fwd", "dgrad", "wgrad", "wgrad_acc"])
    ap.add_argument("--rows", type=int, default=8192, help="rows / tokens of the row-wise kernels (rmsnorm, swiglu, qkv_rope)")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--docs", type=int, default=1)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--non-causal", action="store_true")
    ap.add_argument("--heads", type=int, default=0, help="query heads of the attention benchmark (0: 32, or 16 at head size 256)")
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--library", action="store_true", help="attention: time torch's varlen attention on the same inputs")
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    t = Timer(a.iters, a.warmup, not a.no_flush)
    if a.what == "gemm":
        bench_gemm(t, a.m, a.n, a.k, a.layout)
    elif a.what == "attention":
        hq = a.heads or (16 if a.head_dim == 256 else 32)
        bench_attention(t, a.tokens, a.docs, hq=hq, hkv=a.kv_heads or hq // 4, d=a.head_dim, causal=not a.non_causal,
                        backward=a.backward, library=a.library)
    elif a.what == "rmsnorm":
        bench_rmsnorm(t, rows=a.rows)
    elif a.what == "swiglu":
        bench_swiglu(t, rows=a.rows)
    elif a.what == "qkv_rope":
        bench_qkv_rope(t, tokens=a.rows)
    elif a.what == "ce":
        bench_ce(t)
    elif a.what == "adamw":
        bench_adamw(t)
    elif a.what == "moe":
        bench_moe(t)
    elif a.what == "gemm_wgather":
        bench_gemm_wgather(t, a.m, a.n, a.k)
    elif a.what == "gdn":
        bench_gdn(t, a.tokens, a.docs, heads=a.heads or 32, backward=a.backward)
    elif a.what == "gdn_scan":
        bench_gdn_scan(t, a.tokens, a.docs, reverse=a.backward)
    elif a.what == "conv1d":
        bench_conv1d(t, a.tokens, backward=a.backward)
    elif a.what == "dsa":
        bench_dsa(t, backward=a.backward)
    elif a.what == "fused_adamw":
        bench_fused_adamw(t)
        bench_fused_adamw(t, state=torch.bfloat16)
    elif a.what == "gemm_ag":
        bench_gemm_ag(t, a.m, a.n, a.k, b_mn=a.layout == "dgrad")
    elif a.what == "gelu":
        bench_gelu(t)
    elif a.what == "rope_vision":
        bench_rope_vision(t)
    elif a.what == "layernorm":
        bench_layernorm(t, a.rows if a.rows != 8192 else 28672)
    elif a.what == "gemm_fp8":
        bench_gemm_fp8(t, a.m, a.n, a.k, accumulate=a.layout == "wgrad_acc")
    elif a.what == "linear_fp8":
        bench_linear_fp8(t, a.m, a.n, a.k)
    elif a.what == "gemm_rs_push":
        bench_gemm_rs_push(t, a.m, a.n, a.k, b_mn=a.layout == "dgrad")
    else:
        for layout in ("fwd", "dgrad", "wgrad"):
            bench_gemm(t, 8192, 6144, 4096, layout)
            bench_gemm(t, 8192, 24576, 4096, layout)
            bench_gemm(t, 8192, 4096, 12288, layout)
        bench_gemm(t, 28672, 3456, 1152, "fwd")
        bench_gemm(t, 28672, 4304, 1152, "fwd")
        bench_gemm(t, 4096, 151936, 4096, "fwd")
        for docs in (1, 4, 16):
            bench_attention(t, 8192, docs)
            bench_attention(t, 8192, docs, backward=True)
        bench_attention(t, 16384, 8, hq=16, hkv=16, d=128, causal=False)
        for docs in (1, 16):
            bench_attention(t, 16384, docs, hq=16, hkv=4, d=256)
            bench_attention(t, 16384, docs, hq=16, hkv=4, d=256, backward=True)
        bench_rmsnorm(t)
        bench_swiglu(t)
        bench_qkv_rope(t)
        bench_ce(t)
        bench_adamw(t)
        bench_fused_adamw(t)
        bench_fused_adamw(t, state=torch.bfloat16)
        bench_gemm_ag(t, 8192, 3072, 4096)
        bench_gemm_ag(t, 8192, 2048, 4096, b_mn=True)
        bench_moe(t)
        for docs in (1, 16):
            bench_gdn_scan(t, 16384, docs)
            bench_gdn_scan(t, 16384, docs, reverse=True)
        bench_conv1d(t)
        bench_conv1d(t, backward=True)
        bench_dsa(t)
        bench_dsa(t, backward=True)
    from . import cuda as cu

    cu.check_status()


if __name__ == "__main__":
    main()
