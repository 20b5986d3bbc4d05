"""Headline benchmark: training throughput of the Qwen3-VL-8B-shaped VLM on N B200s.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # the reference stack, same metric/config

Metric: tokens/sec of the WHOLE job (all N GPUs), bf16, synthetic packed multimodal rows of
8192 tokens, random-init weights.  Parallelism: N=1 → single GPU; N>=2 → FSDP x TP = (N/2) x 2
with sequence parallelism (the configuration the baseline names); one packed row per
data-parallel rank per optimizer step, so per-GPU work is fixed as N grows (weak scaling).

Two timings of the same step, both on the device with CUDA events, max over ranks:
  * ``value``: K optimizer steps whose inputs are already on the device;
  * ``e2e``: K steps through ``Trainer.train_step`` — every step copies its batch from pinned host
    memory and reads the loss back.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_SEC_PER_GPU = None  # the reference publishes no tokens/s for this model (plots only)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-vl-8b")
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--ac", default="auto", choices=["auto", "off", "full", "sac"])
    ap.add_argument("--tp", type=int, default=0, help="0 = 1 for one GPU, 2 otherwise")
    ap.add_argument("--no-sp", action="store_true")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel group size (MoE models; data parallel only, tp = 1)")
    ap.add_argument("--ce-chunk", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the number of decoder layers (result is not a bench value)")
    ap.add_argument("--opt-state", default="auto", choices=["auto", "fp32", "bf16"])
    ap.add_argument("--vit-ac", default="auto", choices=["auto", "off", "full"])
    ap.add_argument("--reshard", action="store_true", help="shard parameters and gradients too (ZeRO-3 residency); not the default layout")
    ap.add_argument("--float8", action="store_true",
                    help="FP8 GEMMs for the language model's linear layers (training.float8); not the benchmark of record, which is bf16")
    ap.add_argument("--no-fuse-first-gemm", action="store_true", help="with --reshard: gather every weight by the block's parameter gather")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--sync-debug", action="store_true", help="warn on every host<->device synchronisation inside the end-to-end loop")
    ap.add_argument("--profile", default="", help="write a torch-profiler kernel table of one step to this file (not a bench run)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = sorted(int(float(r[0])) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [int(float(r[1])) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, col in (("hw_slowdown", 3), ("hw_thermal_slowdown", 4), ("sw_thermal_slowdown", 5), ("sw_power_cap", 6)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_config(args, world: int):
    from vlm_training_b200.config import Config

    cfg = Config()
    name = "Qwen3-VL-8B" if "vl" in args.model else ("Qwen3.5-35B-A3B" if "moe" in args.model else
                                                      ("Qwen3.5-9B" if "3.5" in args.model else "Qwen3-8B"))
    cfg.model.model_name, cfg.model.preset = name, args.model
    cfg.model.train_llm = cfg.model.train_mlp = cfg.model.train_vit = True
    t = cfg.training
    tp = args.tp if args.tp else (1 if (world == 1 or args.ep > 1) else 2)
    t.ep_size = args.ep
    t.tp_size, t.sequence_parallel = tp, (tp > 1 and not args.no_sp)
    t.data_parallel = "fsdp"
    t.bfloat16, t.device = True, "cuda"
    t.lr_llm, t.lr_mlp, t.lr_vit, t.weight_decay = 2e-6, 1e-5, 1e-6, 0.01
    t.total_steps, t.warmup_steps, t.save_steps = 10 ** 9, 50, 0
    t.ce_chunk_size = args.ce_chunk
    t.ac_mode = args.ac if args.ac != "auto" else "off"
    # bf16 Adam moments (fp32 master weights kept) at every N: on one GPU they leave room for the decoder's activations
    # of the whole 8.8 B-parameter model without recomputation, and the optimizer pass moves 20 instead of 28 bytes per
    # parameter; the same precision at every N keeps the scaling curve a like-for-like comparison
    t.optimizer_state_dtype = args.opt_state if args.opt_state != "auto" else "bf16"
    t.fused_comm = os.environ.get("VLMT_FUSED_COMM", "1") == "1"
    t.reshard_params = bool(args.reshard)
    t.reshard_fuse_first_gemm = not args.no_fuse_first_gemm
    t.float8 = args.float8
    t.output_dir = "/tmp/vlmt_bench"
    cfg.data.synthetic = "vlm" if "vl" in args.model else "text-loguniform"
    cfg.data.seq_len = args.seq_len
    cfg.data.doc_len_min, cfg.data.doc_len_max = 128, args.seq_len
    cfg.wandb.mode, cfg.wandb.log_topk = "disabled", False
    return cfg


def run_ours(args):
    import torch
    import torch.distributed as dist

    from vlm_training_b200.models import config as mc
    from vlm_training_b200.train.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.layers or "moe" in args.model:
        base = mc._PRESETS[args.model]

        def adjusted():
            c = base()
            if args.layers:
                c.text.num_hidden_layers = args.layers
            if "moe" in args.model:
                c.vision = None   # text rows only: the vision tower of this preset would hold parameters that never get a gradient
            return c
        mc._PRESETS[args.model] = adjusted
    cfg = build_config(args, world)
    tr = Trainer(cfg)
    # activations of the vision tower are kept (no recomputation): on one GPU the step then peaks at about 155 of
    # the 180 GB; "--vit-ac full" trades 9 % of the step time for 21 GB
    vit_ac = args.vit_ac if args.vit_ac != "auto" else "off"
    if tr.model.visual is not None:
        tr.model.visual.ac_mode = vit_ac
    from vlm_training_b200.ops import cuda as cu

    dev = tr.device
    rank = tr.rank

    def barrier():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if not dist.is_initialized():
            return x
        t = torch.tensor([x], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_dp(x: float) -> float:
        if not dist.is_initialized():
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item()) / tr.mesh.tp

    # ---------------------------------------------------------------- device-staged loop
    it = tr.batch_generator()
    # a few distinct rows, already on the device; never more rows than warm-up steps, so every row (and every buffer size
    # that depends on its image mix) has been seen once before the timed region
    staged = [next(it) for _ in range(max(1, min(4, args.steps, args.warmup)))]
    tokens_per_step = float(args.seq_len)

    def one_step(kwargs):
        tr.optimizer.set_requires_gradient_sync(True)
        out = tr.model(**kwargs)
        out.loss.backward()
        tr.optimizer.step()
        tr.optimizer.zero_grad()
        tr.scheduler.step()
        return out.loss.detach()

    # ---------------------------------------------------------------- correctness of the NVLink layer collectives (untimed)
    tp_check = None
    tp_ctx = getattr(tr, "tp_ctx", None)
    if tp_ctx is not None and getattr(tp_ctx, "p2p", None) is not None:
        # one forward + backward on the same row and weights through our own kernels (all-gather fused into the GEMM,
        # GEMM + reduce-scatter) and through torch.distributed's NCCL collectives: loss and gradient norm must agree
        def fwd_bwd_norm():
            tr.optimizer.set_requires_gradient_sync(False)   # no reduction, no update: the local gradients are compared
            out = tr.model(**staged[0])
            out.loss.backward()
            sq = sum(d.flat_grad.float().pow(2).sum() for d in tr.optimizer.domains)
            dist.all_reduce(sq)
            res = (float(out.loss.detach().item()), float(sq.sqrt().item()))
            for d in tr.optimizer.domains:
                d.flat_grad.zero_()
            return res
        p2p = tp_ctx.p2p
        own = fwd_bwd_norm()
        tp_ctx.p2p = None
        lib = fwd_bwd_norm()
        tp_ctx.p2p = p2p
        tr.optimizer.zero_grad()
        tp_check = {"loss_own_kernels": own[0], "loss_nccl": lib[0], "grad_norm_own_kernels": own[1], "grad_norm_nccl": lib[1],
                    "rel_diff_loss": abs(own[0] - lib[0]) / max(abs(lib[0]), 1e-9),
                    "rel_diff_grad_norm": abs(own[1] - lib[1]) / max(abs(lib[1]), 1e-9)}
    for i in range(args.warmup):
        one_step(staged[i % len(staged)])
    barrier()
    if args.profile:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            one_step(staged[0])
            torch.cuda.synchronize()
        if rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(args.profile)), exist_ok=True)
            from torch.autograd import DeviceType

            rows = [e for e in prof.key_averages() if e.device_type == DeviceType.CUDA]
            rows.sort(key=lambda e: -e.self_device_time_total)
            total = sum(e.self_device_time_total for e in rows)
            with open(args.profile, "w") as fh:
                fh.write(f"kernels of one optimizer step, {world} GPU(s), rank 0: {total / 1e3:.1f} ms of device time\n")
                fh.write(f"{'ms':>9} {'share':>7} {'calls':>6}  kernel\n")
                for e in rows[:100]:
                    fh.write(f"{e.self_device_time_total / 1e3:9.3f} {100 * e.self_device_time_total / max(total, 1):6.2f}% {e.count:6d}  {e.key[:150]}\n")
    torch.cuda.reset_peak_memory_stats()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    launches0 = cu.LAUNCHES["count"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        loss = one_step(staged[i % len(staged)])
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    launches = cu.LAUNCHES["count"] - launches0
    peak_mem = torch.cuda.max_memory_allocated() / 2 ** 30
    free_b, total_b = torch.cuda.mem_get_info()
    dev_used = (total_b - free_b) / 2 ** 30   # includes symmetric-memory buffers, which the caching allocator does not count
    global_tokens = sum_over_dp(tokens_per_step)
    value = global_tokens * args.steps / (ms / 1e3)
    cu.check_status()
    # ---------------------------------------------------------------- end-to-end loop (public API)
    e2e = None
    if not args.skip_e2e:
        data_it = tr.batch_generator()
        tr._window = {"tokens": 0, "label_tokens": 0, "samples": 0, "micro": 0, "data_time": 0.0, "h2d_bytes": 0}
        for _ in range(2):
            tr.train_step(data_it)
        tr.flush_metrics()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        got = []
        if args.sync_debug:
            torch.cuda.set_sync_debug_mode("warn")
        t_host = []
        for _ in range(args.steps):
            # every step: H2D of its batch from pinned memory, and a D2H copy of its loss / reductions / status word;
            # the host reads step k's numbers when step k + 1 has been enqueued, so the device never waits for it
            th = time.perf_counter()
            m = tr.train_step(data_it)
            t_host.append(round((time.perf_counter() - th) * 1e3, 1))
            if m is not None:
                got.append(m)
        if args.sync_debug:
            torch.cuda.set_sync_debug_mode("default")
            if rank == 0:
                print(f"host ms per train_step call: {t_host}", file=sys.stderr)
        got.append(tr.flush_metrics())  # the last step's numbers: all K read-backs end inside the timed region
        e1.record()
        barrier()
        assert len(got) == args.steps and all(math.isfinite(m["train/loss"]) for m in got), "a step's loss did not reach the host"
        ms_e2e = max_over_ranks(e0.elapsed_time(e1))
        e2e = {"value": global_tokens * args.steps / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
               "h2d_bytes_per_step": sum(int(m["perf/h2d_bytes"]) for m in got) // args.steps,
               "d2h_bytes_per_step": sum(int(m["perf/d2h_bytes"]) for m in got) // args.steps,
               "losses": [round(float(m["train/loss"]), 4) for m in got[-4:]],
               # where the difference to the device-timed loop comes from: the steps' own device time (CUDA events inside
               # train_step; every step sees a new row with its own image mix) and the share of wall time spent waiting for data
               "device_ms_per_step_by_events": round(1e3 * sum(float(m["perf/step_time"]) for m in got) / len(got), 2),
               "data_wait_pct": round(sum(float(m["perf/data_time_pct"]) for m in got) / len(got), 2)}
    tr.end_run()
    flops_tok = tr.flops_per_token * tr.mesh.tp  # whole-model FLOPs per token
    if rank == 0:
        n = world
        line = {
            "metric": f"tokens/sec (whole job), {cfg.model.model_name}-shaped {'VLM ' if cfg.data.synthetic == 'vlm' else ''}training step", "value": value, "unit": "tokens/s",
            "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (value / n / BASELINE_TOKENS_PER_SEC_PER_GPU) if BASELINE_TOKENS_PER_SEC_PER_GPU else None,
            "dtype": "bf16 with fp8 (e4m3 / e5m2) linear GEMMs in the language model" if args.float8 else "bf16", "data": ("synthetic packed multimodal rows" if cfg.data.synthetic == "vlm" else "synthetic packed text rows")
                                     + ", random-init weights", "impl": "ours",
            "tokens_per_sec_per_gpu": value / n,
            "mfu_vs_measured_sustained": value * flops_tok / n / tr.peak_flops,
            "config": {"model": args.model, "global_batch": int(round(global_tokens / args.seq_len)), "seq_len": args.seq_len,
                       "parallelism": f"fsdp{tr.mesh.dp}xtp{tr.mesh.tp}" + ("+sp" if cfg.training.sequence_parallel else "")
                                      + (f"+ep{args.ep}" if args.ep > 1 else ""),
                       "ac_mode": cfg.training.ac_mode, "optimizer": f"AdamW, fp32 master + {cfg.training.optimizer_state_dtype} moments, sharded over dp", "vit_ac": vit_ac,
                       "l2": "not flushed: every step streams >17 GB of weights, far above the 126 MB L2",
                       "layers_override": args.layers or None, "ce_chunk": args.ce_chunk,
                       "reshard_params": bool(args.reshard)},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "peak_mem_gib": peak_mem, "device_mem_used_gib": dev_used, "tp_path_check": tp_check, "final_loss": float(loss.item()),
        }
        print(json.dumps(line))
    if dist.is_initialized():
        dist.destroy_process_group()


def run_reference(args):
    try:
        from baseline.reference_harness import run
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"baseline harness failed to import: {exc!r}"[:300]}))
        return
    run(args)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
