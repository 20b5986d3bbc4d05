"""The training loop: ``Trainer(cfg).train()``.

Mirrors the reference trainer's surface and order of set-up (reference:
train/train_qwen.py:69-721): process group → mesh → model → (weight surgery) →
device/bf16 → TP → AC → data-parallel engine → data → loop of micro-batches with
fractional gradient accumulation, per-step metrics, periodic DCP checkpoints.

Differences that are deliberate:
* device time is measured with CUDA events (the reference reads ``perf_counter`` without
  a device sync, reference: train/train_qwen.py:537,550);
* gradients are reduced once per optimizer step, not once per micro-batch;
* no host sync inside the step on a GPU: token counts come from the host copy of the batch; the loss, the
  data-parallel reductions and the device status word of step ``k`` travel to pinned host memory by an
  asynchronous copy and are read when step ``k + 1`` has been enqueued (``training.async_metrics``), so the
  metrics of a step are returned one call later and the GPU never idles while the host catches up;
* three optimizer groups as intended (see :mod:`.optimizer`).
"""
from __future__ import annotations

import itertools
import os
import time

import torch
import torch.distributed as dist
from torch.distributed.elastic.multiprocessing.errors import record

from ..config import Config, ModelType, to_flat_dict
from ..data.loader import PrefetchLoader, batch_nbytes, to_device
from ..models import MODEL_CLASSES, ModelConfig
from ..models.init import init_normal_, init_qwen35_, init_qwen3vl_
from ..parallel.ac import apply_ac
from ..parallel.mesh import get_mesh, init_distributed
from ..parallel.tp import apply_tp
from . import checkpoint as ckpt
from .flops import get_dense_model_nparams_and_flops, peak_flops
from .freeze import set_determinism, set_model
from .logger import colors, init_logger, logger
from .metrics import PERF_KEYS, gather_perf, topk_report
from .optimizer import create_optimizer
from .schedulers import accumulation_pattern, build_scheduler

_FAMILY = {ModelType.QWEN3_5: "qwen3_5", ModelType.QWEN3_VL: "qwen3_vl", ModelType.QWEN3_TEXT: "qwen3_text"}


def select_model_class(model_type: ModelType):
    return MODEL_CLASSES[_FAMILY[model_type]]


class Trainer:
    @record  # a failure during set-up lands in torchrun's error file (reference: train/train_qwen.py:17,71)
    def __init__(self, cfg: Config):
        self.cfg = cfg
        t = cfg.training
        self.rank, self.world, self.device = init_distributed(t.backend, t.device)
        init_logger(self.rank)
        self.mesh = get_mesh(t.tp_size, self.device)
        logger.info(f"{self.mesh}")
        self.debug = bool(os.environ.get("DEBUG"))
        set_determinism(t.seed)  # one seed for every rank: weights are drawn identically without a broadcast
        if self.device.type == "cuda":
            # float32 library matmuls (the intra-chunk part of the gated delta rule) may use TF32 tensor cores, as in
            # the reference trainer (train/train_qwen.py:65-66)
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
        self.wandb = self._init_wandb()

        # ---------------- model
        self.model_type = ModelType.from_name(cfg.model.model_name if cfg.model.model_name != "NULL" else cfg.model.preset)
        cls = select_model_class(self.model_type)
        dtype = torch.bfloat16 if (t.bfloat16 and self.device.type == "cuda") else torch.float32
        if t.model_dir not in ("", "NULL") and os.path.isdir(t.model_dir):
            model, mcfg = cls.from_pretrained(t.model_dir, dtype=dtype, device="cpu", load_vision=not t.load_vision_model)
        else:
            if not cfg.model.preset:
                raise ValueError("training.model_dir is not a snapshot directory and model.preset is empty")
            mcfg = ModelConfig.preset(cfg.model.preset)
            if cfg.model.dsa:
                mcfg.text.dsa, mcfg.text.dsa_topk = True, cfg.model.dsa_topk
            model = cls.from_config(mcfg, dtype=dtype, device=self.device, init=False)
            init_normal_(model, 0.02, seed=t.seed)
        self.model_config = mcfg
        self.seq_len = int(cfg.data.seq_len)
        self.nparams, flops_token = get_dense_model_nparams_and_flops(mcfg, model, self.seq_len)
        self.flops_per_token = flops_token / t.tp_size  # per GPU, as the reference divides (train/train_qwen.py:140)
        self.peak_flops = peak_flops()
        if t.load_text_model:
            from ..utils.surgery import load_text_model

            load_text_model(model, t.text_model_dir)
        if t.load_vision_model:
            from ..utils.surgery import load_vision_model

            load_vision_model(model, t.vision_model_dir)
        if t.random_init:
            (init_qwen35_ if self.model_type is ModelType.QWEN3_5 else init_qwen3vl_)(model, seed=42)
        model = model.to(self.device)
        model.ce_chunk_size = t.ce_chunk_size
        set_model(model, cfg.model.train_llm, cfg.model.train_mlp, cfg.model.train_vit)
        # ---------------- parallelism (order matters: TP → AC → data parallel)
        tp_backend = "p2p" if (t.fused_comm and self.device.type == "cuda" and t.tp_size > 1) else "dist"
        self.tp_ctx = apply_tp(model, self.mesh, sequence_parallel=t.sequence_parallel, backend=tp_backend)
        if getattr(self.tp_ctx, "p2p", None) is not None:
            # largest message of the layer collectives: a gathered [T, hidden] activation gradient, or the vision
            # features of a row whose tokens are all image tokens (merged + DeepStack features side by side)
            n_feat = (1 + len(mcfg.vision.deepstack_visual_indexes)) * mcfg.vision.out_hidden_size if mcfg.vision is not None else 0
            self.tp_ctx.p2p.reserve(self.seq_len * max(mcfg.text.hidden_size, n_feat))
        if t.ep_size > 1:
            from ..parallel.ep import apply_ep

            self.ep_ctx = apply_ep(model, self.mesh, t.ep_size, fused=t.fused_comm and self.device.type == "cuda")
        apply_ac(model, t.ac_mode)
        if t.float8:
            from ..parallel.float8 import apply_float8

            apply_float8(model)
        self.model = model
        self.optimizer = self.create_optimizer()
        self.scheduler = build_scheduler(self.optimizer, t.scheduler_type, t.total_steps, t.warmup_steps,
                                         wsd_decay_ratio=t.wsd_decay_ratio, min_lr_ratio=t.min_lr_ratio)
        # ---------------- data
        self.loader = self._build_loader()
        self.accum_cycle = itertools.cycle(accumulation_pattern(t.tpi_multiplier))
        self.accum_target = next(self.accum_cycle)
        # ---------------- counters
        self.global_step = 0
        self.tokens_seen = 0
        self.tokens_seen_assistant = 0
        self.samples_seen = 0
        self._window = {"tokens": 0, "label_tokens": 0, "samples": 0, "micro": 0, "data_time": 0.0, "h2d_bytes": 0}
        self._last_log = time.perf_counter()
        self._pending = None
        self._cprofile = None
        self._last_perf = None
        self._flushed = []  # metrics resolved by a flush (checkpoint, end of run) that no train_step call returned
        # deferred metrics need pinned memory and events, so they exist on a GPU only
        self.async_metrics = bool(t.async_metrics) and self.device.type == "cuda"
        logger.info(f"model {cfg.model.model_name or cfg.model.preset}: {self.nparams / 1e9:.3f} B parameters, "
                    f"{self.flops_per_token / 1e9:.2f} GFLOP/token/GPU, mode {t.data_parallel} x tp{t.tp_size}")

    # ------------------------------------------------------------------ set-up helpers
    def _init_wandb(self):
        w = self.cfg.wandb
        if w.mode == "disabled" or self.rank != 0:
            return None
        try:
            import wandb

            os.environ.setdefault("WANDB_MODE", w.mode)
            return wandb.init(project=w.project_name, entity=w.entity_name or None, name=w.run_name,
                              config=to_flat_dict(self.cfg))
        except Exception as exc:  # logging must never take the run down
            logger.warning(f"wandb disabled: {exc}")
            return None

    def create_optimizer(self):
        t = self.cfg.training
        fused = t.fused_comm and self.device.type == "cuda" and self.world > 1
        return create_optimizer(self.model, t, self.mesh, fused_comm=fused)

    def _build_loader(self):
        from ..data.loader import WorkerPool, make_dataset

        d = self.cfg.data
        args = (d, self.cfg.training, self.model_config, self.mesh.dp_rank, self.mesh.dp)
        if int(getattr(d, "worker_processes", 0)) > 0:
            ds = WorkerPool(args, int(d.worker_processes), depth=max(2, d.num_workers))
        else:
            ds = make_dataset(*args)
        pixel_dtype = next(self.model.parameters()).dtype
        transfer = lambda b: to_device(b, self.model_config, self.device, pixel_dtype=pixel_dtype)
        return PrefetchLoader(ds, depth=max(2, d.num_workers), transfer=transfer, device=self.device)

    # ------------------------------------------------------------------ data
    def batch_generator(self):
        """Yields model keyword arguments on the device and accounts tokens from the host copy."""
        while True:
            t0 = time.perf_counter()
            try:
                batch = next(self.loader)
            except StopIteration:
                return
            if "kwargs" in batch:  # the loader thread already copied the batch to the device
                meta, kwargs = batch["meta"], batch["kwargs"]
            else:
                meta = {"n_tokens": int(batch["input_ids"].numel()), "n_label": int((batch["labels"] != -100).sum()),
                        "n_docs": int(batch["cu_seqlens"].numel()) - 1, "h2d_bytes": batch_nbytes(batch)}
                kwargs = to_device(batch, self.model_config, self.device, pixel_dtype=next(self.model.parameters()).dtype)
            self._window["tokens"] += meta["n_tokens"]
            self._window["label_tokens"] += meta["n_label"]
            self._window["samples"] += meta["n_docs"]
            self._window["h2d_bytes"] += meta["h2d_bytes"]
            self._window["data_time"] += time.perf_counter() - t0
            yield kwargs

    # ------------------------------------------------------------------ one micro-batch
    def train_step(self, data_iterator) -> dict | None:
        """One micro-batch; runs the optimizer when the accumulation target is reached and then
        returns the step's metrics (else None).  Raises StopIteration when data runs out."""
        t = self.cfg.training
        batch = next(data_iterator)
        last = self._window["micro"] + 1 >= self.accum_target
        self.optimizer.set_requires_gradient_sync(last)
        if self._window["micro"] == 0 and self.device.type == "cuda":
            self._ev_start = torch.cuda.Event(enable_timing=True)
            self._ev_fb = torch.cuda.Event(enable_timing=True)
            self._ev_end = torch.cuda.Event(enable_timing=True)
            self._ev_start.record()
        with torch.profiler.record_function("forward_pass"):
            out = self.model(**batch)
        loss = out.loss / self.accum_target
        with torch.profiler.record_function("backward_pass"):
            loss.backward()
        self._loss_acc = out.loss.detach() if self._window["micro"] == 0 else self._loss_acc + out.loss.detach()
        self._window["micro"] += 1
        if not last:
            return None
        if self.device.type == "cuda":
            self._ev_fb.record()
        with torch.profiler.record_function("optimizer_step"):
            self.optimizer.step()
            self.optimizer.zero_grad()
        self.scheduler.step()
        self.global_step += 1
        if self.device.type == "cuda":
            self._ev_end.record()
        metrics = self._finish_step()
        self.accum_target = next(self.accum_cycle)
        return metrics

    def _finish_step(self) -> dict | None:
        """Close the accumulation window: enqueue the step's reductions and read-back, then return the metrics of the
        newest step whose numbers have reached the host (this step when metrics are synchronous, the previous one
        when they are deferred, ``None`` on the first deferred call)."""
        w = self._window
        now = time.perf_counter()
        pend = {"window": w, "wall": now - self._last_log, "step": self.global_step,
                "lr": self.optimizer.param_groups[0]["lr"]}
        self._last_log = now
        cuda = self.device.type == "cuda"
        # the previous step first: its numbers have long arrived, and its timings feed this step's straggler table
        done = None
        if self._pending is not None:
            done, self._pending = self._resolve(self._pending), None
        loss_local = (self._loss_acc / w["micro"]).double().reshape(1)
        if cuda:
            pend.update(ev_start=self._ev_start, ev_fb=self._ev_fb, ev_end=self._ev_end)
            pend["peak_mem"] = torch.cuda.max_memory_allocated() / 2 ** 30
            torch.cuda.reset_peak_memory_stats()
        # [loss, tokens, label tokens, samples | loss (max) | device status word | straggler table]: the collectives
        # run over the data-parallel group (the table over all ranks) with no host read in between
        counts = torch.tensor([w["tokens"], w["label_tokens"], w["samples"]], dtype=torch.float64)
        if cuda:
            counts = counts.pin_memory().to(self.device, non_blocking=True)
        vec = torch.cat([loss_local, counts])
        mx = loss_local.clone()
        n = 1
        if dist.is_initialized() and self.mesh.dp > 1:
            dist.all_reduce(vec, op=dist.ReduceOp.SUM, group=self.mesh.dp_group)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.mesh.dp_group)
            n = self.mesh.dp
        parts = [vec, mx]
        if cuda:
            from ..ops import cuda as cu

            parts.append(cu.status_word().double())
        else:
            parts.append(torch.zeros(1, dtype=torch.float64))
        want_topk = self.cfg.wandb.log_topk and self.world > 1
        if want_topk and not self.async_metrics:
            pend["topk_now"] = True  # synchronous metrics rank the step itself, after its timings are known
        elif want_topk and self._last_perf is not None:
            table = torch.tensor(self._last_perf, dtype=torch.float64)
            if cuda:
                table = table.pin_memory().to(self.device, non_blocking=True)
            gathered = torch.empty(self.world * table.numel(), dtype=torch.float64, device=self.device)
            dist.all_gather_into_tensor(gathered, table)
            parts.append(gathered)
        packed = torch.cat(parts)
        if cuda:
            host = torch.empty(packed.numel(), dtype=torch.float64, pin_memory=True)
            host.copy_(packed, non_blocking=True)  # the step's device -> host read
            pend["ready"] = torch.cuda.Event()
            pend["ready"].record()
        else:
            host = packed
        pend["host"], pend["dp"] = host, n
        self._window = {"tokens": 0, "label_tokens": 0, "samples": 0, "micro": 0, "data_time": 0.0, "h2d_bytes": 0}
        self._pending = pend
        if not self.async_metrics:
            return self.flush_metrics()
        return done

    def flush_metrics(self) -> dict | None:
        """Wait for the newest step's numbers and return its metrics (``None`` if every step has been reported).
        Called before a checkpoint is written and at the end of the run; raises if a kernel of the step reported a
        bounded wait that ran out."""
        pend, self._pending = self._pending, None
        return self._resolve(pend) if pend is not None else None

    def _resolve(self, pend: dict) -> dict:
        w = pend["window"]
        if "ready" in pend:
            pend["ready"].synchronize()  # long complete unless this is a flush
            step_time = pend["ev_start"].elapsed_time(pend["ev_end"]) / 1e3
            fwd_bwd = pend["ev_start"].elapsed_time(pend["ev_fb"]) / 1e3
        else:
            step_time = fwd_bwd = pend["wall"]
        vals = pend["host"].tolist()
        loss_sum, tok_sum, lab_sum, samp_sum, loss_max, status = vals[:6]
        if int(status) != 0:
            from ..ops import cuda as cu, status as st

            cu.status_word().zero_()
            raise RuntimeError(f"step {pend['step']}: a kernel gave up on a bounded wait: {st.describe(int(status))} "
                               f"(status {int(status)}); the optimizer state of this step may be incomplete")
        if self.device.type == "cuda" and self.world > 1:
            from ..parallel import symm

            if symm.guards_enabled():
                symm.check_guards()   # debug mode: canary bands around every peer-visible buffer
        self.tokens_seen += int(tok_sum)
        self.tokens_seen_assistant += int(lab_sum)
        self.samples_seen += int(samp_sum)
        tps = w["tokens"] / max(step_time, 1e-9)
        tflops = self.flops_per_token * self.seq_len * w["micro"] / max(step_time, 1e-9) / 1e12
        mfu = tflops * 1e12 / self.peak_flops
        m = {"train/loss": loss_sum / pend["dp"], "train/max_loss": loss_max, "train/tokens_seen": self.tokens_seen,
             "train/assistant_tokens_seen": self.tokens_seen_assistant, "train/num_samples": samp_sum,
             "train/lr": pend["lr"],
             "train/batch_efficiency": w["tokens"] / max(1, w["micro"] * self.seq_len),
             "perf/tokens_per_second": tps, "perf/data_time_pct": 100.0 * w["data_time"] / max(pend["wall"], 1e-9),
             "perf/step_time": step_time, "perf/fwd_bwd_time": fwd_bwd, "perf/tflops_per_second": tflops, "perf/mfu": mfu,
             "perf/peak_mem_gib": pend.get("peak_mem", 0.0), "perf/h2d_bytes": w["h2d_bytes"],
             "perf/d2h_bytes": pend["host"].numel() * pend["host"].element_size(), "step": pend["step"]}
        self._last_perf = [tps, step_time, fwd_bwd, tflops, mfu, pend.get("peak_mem", 0.0)]
        if pend.get("topk_now"):
            m.update(topk_report(gather_perf(self._last_perf, self.device), self.cfg.wandb.top_k))
        elif len(vals) > 6:
            # deferred metrics: the ranking was gathered with this step's read-back and describes the step before it
            table = torch.tensor(vals[6:], dtype=torch.float32).view(self.world, len(PERF_KEYS))
            m.update(topk_report(table, self.cfg.wandb.top_k))
        self.log(m)
        return m

    def log(self, m: dict):
        if self.rank != 0:
            return
        if m["step"] % max(1, self.cfg.training.log_every) == 0:
            c = colors()
            logger.info(f"{c.cyan}step {m['step']:>6}{c.reset} loss {c.yellow}{m['train/loss']:.4f}{c.reset} "
                        f"tps {m['perf/tokens_per_second']:,.0f} mfu {100 * m['perf/mfu']:.1f}% "
                        f"tflops {m['perf/tflops_per_second']:.1f} step {m['perf/step_time'] * 1e3:.1f} ms "
                        f"fwd+bwd {m['perf/fwd_bwd_time'] * 1e3:.1f} ms data {m['perf/data_time_pct']:.1f}% "
                        f"nsamples {int(m['train/num_samples'])} batch_util {m['train/batch_efficiency']:.3f}")
        if self.wandb is not None:
            self.wandb.log({k: v for k, v in m.items() if k != "step"}, step=m["step"])

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self):
        m = self.flush_metrics()  # counters are final and the device status word of the last step has been checked
        if m is not None:
            self._flushed.append(m)
        with self.optimizer.all_resident():   # sharded parameters are gathered for the model's state dict
            return ckpt.save_checkpoint(self.cfg.training.output_dir, self.global_step, self.model, self.optimizer, self.scheduler,
                                        {"tokens_seen": self.tokens_seen, "tokens_seen_assistant": self.tokens_seen_assistant},
                                        tp_rank=self.mesh.tp_rank)

    def load_checkpoint(self, step: int):
        with self.optimizer.all_resident():
            c = ckpt.load_checkpoint(self.cfg.training.output_dir, step, self.model, self.optimizer, self.scheduler,
                                     tp_rank=self.mesh.tp_rank)
        self.global_step = c["step"]
        self.tokens_seen, self.tokens_seen_assistant = c["tokens_seen"], c["tokens_seen_assistant"]

    def may_save(self):
        s = self.cfg.training.save_steps
        if s > 0 and self.global_step > 0 and self.global_step % s == 0:
            self.save_checkpoint()

    # ------------------------------------------------------------------ loop
    def train(self):
        t = self.cfg.training
        data_iterator = self.batch_generator()
        if t.resume_checkpoint:
            step = ckpt.latest_step(t.output_dir)
            if step is None:
                raise FileNotFoundError(f"resume_checkpoint is set but {t.output_dir} holds no checkpoint")
            self.load_checkpoint(step)
        prof = self._profiler()
        history = []
        try:
            with prof if prof is not None else _Null():
                while self.global_step < t.total_steps:
                    before = self.global_step
                    try:
                        m = self.train_step(data_iterator)
                    except StopIteration:
                        logger.info("data exhausted: writing the final checkpoint")
                        self.save_checkpoint()
                        break
                    if prof is not None:
                        prof.step()
                    if m is not None:
                        history.append(m)
                    if self.global_step != before:  # an optimizer step was taken
                        self._cprofile_window()
                        self.may_save()
                    history.extend(self._flushed)
                    self._flushed.clear()
        finally:
            self.end_run()
        history.extend(self._flushed)
        self._flushed.clear()
        return history

    def _cprofile_window(self):
        """``DEBUG=1``: profile the host side of optimizer steps ``cprofile_start`` .. ``cprofile_stop`` with cProfile
        and write the 50 most expensive call sites by cumulative time to ``cprofile_rank_{r}.txt`` in the output
        directory (reference: train/train_qwen.py:607-615,667-694)."""
        if not self.debug:
            return
        t = self.cfg.training
        if self.global_step == t.cprofile_start and self._cprofile is None:
            import cProfile

            self._cprofile = cProfile.Profile()
            self._cprofile.enable()
        elif self.global_step >= t.cprofile_stop and self._cprofile is not None:
            self._dump_cprofile()

    def _dump_cprofile(self):
        import io
        import pstats

        prof, self._cprofile = self._cprofile, None
        prof.disable()
        buf = io.StringIO()
        pstats.Stats(prof, stream=buf).sort_stats("cumulative").print_stats(50)
        os.makedirs(self.cfg.training.output_dir, exist_ok=True)
        with open(os.path.join(self.cfg.training.output_dir, f"cprofile_rank_{self.rank}.txt"), "w") as fh:
            fh.write(buf.getvalue())

    def _profiler(self):
        """``DEBUG=1``: torch profiler (wait 10, warm-up 2, active 2) writing a chrome trace and a
        key-averages table per rank into the output directory (reference: train/train_qwen.py:641-666)."""
        if not self.debug:
            return None
        out = self.cfg.training.output_dir
        os.makedirs(out, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU]
        if self.device.type == "cuda":
            acts.append(torch.profiler.ProfilerActivity.CUDA)

        def on_ready(p):
            p.export_chrome_trace(os.path.join(out, f"trace_rank_{self.rank}_step_{self.global_step}.json"))
            with open(os.path.join(out, f"trace_rank_{self.rank}_step_{self.global_step}_summary.txt"), "w") as fh:
                fh.write(p.key_averages(group_by_stack_n=5).table(sort_by="self_cuda_time_total" if self.device.type == "cuda"
                                                                  else "self_cpu_time_total", row_limit=40))
        return torch.profiler.profile(activities=acts, schedule=torch.profiler.schedule(wait=10, warmup=2, active=2, repeat=1),
                                      on_trace_ready=on_ready, record_shapes=True, with_stack=True)

    def end_run(self):
        self.loader.close()
        if self._cprofile is not None:  # the run ended inside the window
            self._dump_cprofile()
        try:
            m = self.flush_metrics()  # also checks the device status word of the last step
            if m is not None:
                self._flushed.append(m)
        finally:
            if self.wandb is not None:
                self.wandb.finish()
        if self.device.type == "cuda":
            from ..ops import cuda as cu

            cu.check_status()


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


@record
def main(argv=None):
    import sys

    from ..config import ConfigManager

    cfg = ConfigManager(Config).parse_args(sys.argv[1:] if argv is None else argv)
    trainer = Trainer(cfg)
    try:
        trainer.train()
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()
