"""Timings of the fused compute + collective kernels on N GPUs of one node, against their roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m vlm_training_b200.parallel.microbench_comm [--tokens 8192] [--hidden 4096] [--inter 12288] [--iters 20]

Every rank times with CUDA events on its own stream after a barrier; the reported time is the MAX over ranks of the
per-rank medians.  Roofline of a path = the slower of (FLOPs / measured bf16 GEMM peak) and (bytes that must cross
NVLink per GPU and direction / link bandwidth); the printed fraction is that bound divided by the measured time.
GEMM peak and copy bandwidth come from ``MEASURED_PEAKS.json`` (else 1590 TFLOP/s, 6650 GB/s); the link bandwidth
is the measured peer-copy rate of this machine type, 770 GB/s per direction (900 nominal).

Paths (tensor-parallel group = all ranks):
  wgather_gemm parameter all-gather -> GEMM in one kernel: the weight's shards are pulled from their owners into the local
               bucket by two extra warps per CTA while the first tiles run on this rank's own part
  ag_gemm      all-gather -> GEMM in one kernel (column-parallel forward: qkv, gate/up; gather of dY + input
               gradient of the row-parallel linears: o_proj, down_proj)
  gemm_rs      GEMM -> reduce-scatter: tile stores into the owner's memory from the epilogue, then the local sum
  pull_gather  all-gather as peer loads (vision features, non-GEMM gathers)
  pull_reduce  reduce-scatter as peer loads with fp32 accumulation
  rs_adamw_ag  gradient reduce-scatter + AdamW + parameter all-gather in one kernel, per 256 MB bucket
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _peaks():
    from ..ops.microbench import peaks

    return peaks()


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _report(rank, name, shape, ms, flops, link_bytes, hbm_bytes=0.0):
    pk = _peaks()
    t_compute = flops / (pk["tflops"] * 1e12) * 1e3
    t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e3
    t_hbm = hbm_bytes / (pk["gbs"] * 1e9) * 1e3
    bound = max(t_compute, t_link, t_hbm)
    kind = "compute" if bound == t_compute else ("nvlink" if bound == t_link else "hbm")
    if rank == 0:
        print(json.dumps({"path": name, "shape": shape, "ms": round(ms, 4), "roofline_ms": round(bound, 4), "bound": kind,
                          "fraction_of_roofline": round(bound / ms, 3), "tflops": round(flops / ms / 1e9, 1) if flops else None,
                          "link_gbs": round(link_bytes / ms / 1e6, 1) if link_bytes else None, "peaks": pk["source"]}), flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--qkv", type=int, default=6144)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--bucket-mb", type=float, default=256.0)
    a = ap.parse_args(argv)

    from ..ops import cuda as cu
    from . import symm
    from .mesh import init_distributed
    from .p2p import P2PComm

    rank, world, dev = init_distributed("nccl", "cuda")
    if world < 2:
        raise SystemExit("run under torchrun with at least 2 ranks")
    comm = P2PComm(dist.group.WORLD, dev)
    T, H, I, Q = a.tokens, a.hidden, a.inter, a.qkv
    R = T // world
    r = lambda *s: (torch.randn(*s, device=dev) * 0.05).bfloat16()
    frac = (world - 1) / world

    # ---- all-gather -> GEMM
    x_loc = r(R, H)
    for name, w, b_mn, site in (("ag_gemm qkv fwd", r(Q // world, H), False, object()),
                                ("ag_gemm gate_up fwd", r(2 * I // world, H), False, object()),
                                ("ag_gemm o_proj dgrad", r(H, (Q * 2 // 3) // world), True, None),
                                ("ag_gemm down dgrad", r(H, I // world), True, None)):
        n_out = w.shape[1] if b_mn else w.shape[0]
        comm.begin_microbatch()
        ms = _time(lambda: comm.gemm_all_gather(x_loc, w, b_mn=b_mn, site=site), a.iters)
        _report(rank, name, [T, n_out, H], ms, 2.0 * T * n_out * H, frac * T * H * 2)

    # ---- GEMM -> reduce-scatter
    for name, x, w, b_mn in (("gemm_rs o_proj fwd", r(T, (Q * 2 // 3) // world), r(H, (Q * 2 // 3) // world), False),
                             ("gemm_rs down fwd", r(T, I // world), r(H, I // world), False),
                             ("gemm_rs qkv dgrad", r(T, Q // world), r(Q // world, H), True),
                             ("gemm_rs gate_up dgrad", r(T, 2 * I // world), r(2 * I // world, H), True)):
        k = x.shape[1]
        ms = _time(lambda: comm.gemm_reduce_scatter(x, w, b_mn=b_mn), a.iters)
        _report(rank, name, [T, H, k], ms, 2.0 * T * H * k, frac * T * H * 2, hbm_bytes=(world + 1) * R * H * 2)

    # ---- parameter all-gather -> GEMM (the first GEMM of a block whose parameters are sharded over the ranks)
    for name, n_out in (("wgather_gemm qkv", Q), ("wgather_gemm gate_up", 2 * I)):
        shard_n = (n_out * H // world + 8 * world) // 8 * 8
        shard = symm.symmetric_zeros(shard_n, torch.bfloat16, dev, dist.group.WORLD)
        shard.normal_(0, 0.05)
        bucket = torch.zeros(shard_n * world, dtype=torch.bfloat16, device=dev)
        w_view = bucket[:n_out * H].view(n_out, H)
        x_full = r(T, H)
        out = torch.empty(T, n_out, dtype=torch.bfloat16, device=dev)
        sync = torch.zeros(2 * world, dtype=torch.int32, device=dev)
        ptrs = symm.peer_ptrs(shard)
        torch.cuda.synchronize()
        dist.barrier()
        ep = [0]

        def wg():
            ep[0] += 1
            cu._C.gemm_wgather(x_full, w_view, out, None, bucket, ptrs, shard_n, rank, sync, ep[0])
        ms = _time(wg, a.iters)
        _report(rank, name, [T, n_out, H], ms, 2.0 * T * n_out * H, frac * n_out * H * 2)

    # ---- plain peer collectives
    x = r(R, H)
    ms = _time(lambda: comm.all_gather_rows(x), a.iters)
    _report(rank, "pull_gather", [R, H], ms, 0.0, frac * T * H * 2)
    y = r(T, H)
    ms = _time(lambda: comm.reduce_scatter_rows(y), a.iters)
    _report(rank, "pull_reduce", [T, H], ms, 0.0, frac * T * H * 2)

    # ---- reduce-scatter + AdamW + all-gather, one bucket
    n = int(a.bucket_mb * (1 << 20) / 2) // (8 * world) * (8 * world)
    grads = symm.symmetric_zeros(n, torch.bfloat16, dev, dist.group.WORLD)
    params = symm.symmetric_zeros(n, torch.bfloat16, dev, dist.group.WORLD)
    grads.normal_()
    torch.cuda.synchronize()
    dist.barrier()
    shard = n // world
    lo, hi = rank * shard, (rank + 1) * shard
    for sdt, sname in ((torch.float32, "fp32 moments"), (torch.bfloat16, "bf16 moments")):
        master = torch.zeros(shard, device=dev)
        m1, m2 = torch.zeros(shard, device=dev, dtype=sdt), torch.zeros(shard, device=dev, dtype=sdt)
        for mc, mname in ((False, "peer ld/st"), (True, "multimem")):
            g_mc, p_mc = (symm.multicast_ptr(grads), symm.multicast_ptr(params)) if mc else (0, 0)
            if mc and not (g_mc and p_mc):
                continue
            fn = lambda: cu._C.fused_rs_adamw_ag(symm.peer_ptrs(grads), symm.peer_ptrs(params), g_mc, p_mc, world, lo, hi, master, m1,
                                                 m2, 0, 1e-5, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0 / world, False)
            ms = _time(fn, a.iters)
            sb = 4 if sdt == torch.float32 else 2
            # per GPU and direction: its shard's gradients read from every peer plus the peers' parameter shards written
            # into its memory; HBM: gradients and parameters of the whole bucket once each, the shard's state read + written
            _report(rank, f"rs_adamw_ag {sname}, {mname}", [n], ms, 0.0, 2.0 * (world - 1) * shard * 2,
                    hbm_bytes=shard * (4.0 * world + 8 + 4 * sb))
    cu.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
