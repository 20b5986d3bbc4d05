"""Runs the reference stack (VLR-CVC/vlm-training, unmodified copy under ``baseline/_ref``) on the
headline benchmark: same metric, model shape, data and timing as ``bench.py``'s own arm.

What runs is the reference's own code: its ``Qwen3VLForCausalLM`` model, ``get_mesh`` /
``apply_tp`` / ``apply_ac`` / ``apply_fsdp`` (torch FSDP2 + DTensor TP over NCCL, FlashAttention-2
behind ``varlen_attn``, cuBLAS), bf16 cast, ``torch.optim.AdamW(foreach=True)`` with its parameter
grouping, autocast forward, full-logits cross entropy — in the order of its trainer
(reference: train/train_qwen.py:159-210, 273-328, 534-557).  What is substituted, because the
packages are not installable offline and the trainer class hard-wires them:
  * ``torchao`` / ``megatron.energon`` / ``causal_conv1d``: empty stub modules so
    ``train.infra`` imports (none of them is on the Qwen3-VL code path);
  * the HF snapshot + energon dataset: random-init weights (std 0.02) from a config of the
    benchmark shape, and the same synthetic packed rows this framework's arm uses.
"""
from __future__ import annotations

import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _stub_modules():
    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    if "torchao" not in sys.modules:
        try:
            import torchao.float8  # noqa: F401
        except Exception:
            mod("torchao")
            mod("torchao.float8", convert_to_float8_training=lambda *a, **k: None, Float8LinearConfig=object)
    try:
        import megatron.energon  # noqa: F401
    except Exception:
        mod("megatron")
        mod("megatron.energon")
    try:
        import causal_conv1d  # noqa: F401
    except Exception:
        mod("causal_conv1d", causal_conv1d_fn=None)


def run(args):
    if not os.path.isdir(os.path.join(REF, "models")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not hold the reference sources"}))
        return
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REF)
    _stub_modules()
    try:
        from models.qwen3_vl.model import (Qwen3VLConfig, Qwen3VLForCausalLM, Qwen3VLTextConfig, Qwen3VLVisionConfig)
        from train.config import ModelType
        from train.infra import ACConfig, apply_ac, apply_fsdp, apply_tp, compile_model, get_dp_group, get_mesh, get_tp_group
    except Exception as exc:
        print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {exc!r}"[:300]}))
        return

    # this framework is used only for the synthetic data stream and the timing helpers
    sys.path.insert(0, os.path.dirname(HERE))
    from bench import ClockSampler
    from vlm_training_b200.data.synthetic import SyntheticDataset, SyntheticSpec
    from vlm_training_b200.models.config import ModelConfig

    for k, v in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29517")):
        os.environ.setdefault(k, v)  # a plain `python bench.py --impl reference` is a one-rank job
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)  # the reference always initialises NCCL (train/train_qwen.py:79)
    tp = args.tp if args.tp else (1 if world == 1 else 2)
    note = None
    if tp > 1 and os.environ.get("REF_FORCE_TP", "0") != "1":
        # The reference's Qwen3-VL tensor-parallel plan does not run with its own Qwen3-VL model: q/k come out of the
        # column-parallel projections as DTensors while cos/sin stay plain tensors, and `apply_rope` raises
        # "aten.mul.Tensor got mixed torch.Tensor and DTensor" (train/infra.py:432-452 prepares a `hidden_states`
        # keyword the model never passes; observed on 2 GPUs).  The reference's working multi-GPU layout for this
        # model is FSDP over all ranks, which is what is measured instead.
        note = "reference TP plan for Qwen3-VL fails (mixed Tensor/DTensor in apply_rope); measured with its FSDP-only layout"
        tp = 1

    class TrainingArgs:
        tp_size = tp
        async_tp = True

    mesh = get_mesh(TrainingArgs, world)
    tp_group, dp_group = get_tp_group(mesh), get_dp_group(mesh)
    dp_rank, dp_size = dp_group.get_local_rank(), dp_group.size()

    ours = ModelConfig.preset(args.model)
    t, v = ours.text, ours.vision
    n_layers = args.layers or t.num_hidden_layers
    cfg = Qwen3VLConfig(
        text=Qwen3VLTextConfig(vocab_size=t.vocab_size, hidden_size=t.hidden_size, intermediate_size=t.intermediate_size,
                               num_hidden_layers=n_layers, num_attention_heads=t.num_attention_heads,
                               num_key_value_heads=t.num_key_value_heads, head_dim=t.head_dim,
                               max_position_embeddings=t.max_position_embeddings, rms_norm_eps=t.rms_norm_eps,
                               rope_theta=t.rope_theta, tie_word_embeddings=False, mrope_section=list(t.mrope_section),
                               mrope_interleaved=True),
        vision=Qwen3VLVisionConfig(depth=v.depth, hidden_size=v.hidden_size, intermediate_size=v.intermediate_size,
                                   num_heads=v.num_heads, in_channels=v.in_channels, patch_size=v.patch_size,
                                   temporal_patch_size=v.temporal_patch_size, spatial_merge_size=v.spatial_merge_size,
                                   num_position_embeddings=v.num_position_embeddings, out_hidden_size=v.out_hidden_size,
                                   hidden_act=v.hidden_act, deepstack_visual_indexes=list(v.deepstack_visual_indexes)),
        image_token_id=ours.image_token_id, video_token_id=ours.video_token_id,
        vision_start_token_id=ours.vision_start_token_id, vision_end_token_id=ours.vision_end_token_id,
        tie_word_embeddings=False)
    torch.manual_seed(42)
    with torch.device(dev):
        model = Qwen3VLForCausalLM(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
    model.train()
    model = model.to(torch.bfloat16)
    if tp > 1:
        apply_tp(model, ModelType.Qwen3_vl, tp_group, True)
    ac_mode = os.environ.get("REF_AC", "off" if args.ac == "auto" else args.ac)
    if ac_mode != "off":
        apply_ac(model.model.language_model, ACConfig(enabled=True, full=(ac_mode == "full")), model_compile_enabled=False)
    apply_fsdp(ModelType.Qwen3_vl, model, mesh=dp_group)
    # torch.compile is the reference's default (train/config.py:110) and is applied after FSDP as its trainer does
    # (train/train_qwen.py:196-209); REF_COMPILE=0 runs it eagerly.  If compilation fails on this box the harness
    # re-executes itself eagerly and says so in its output.
    compiled = os.environ.get("REF_COMPILE", "1") == "1"
    if compiled:
        compile_model(model)
    # optimizer exactly as the reference builds it (every non-merger parameter lands in the lr_mlp group)
    mlp_params, vision_params, llm_params = [], [], []
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        if "visual.merger" in n:
            mlp_params.append(p)
        elif "visual.deepstack_merger_list":
            mlp_params.append(p)
    groups = [{"params": mlp_params, "lr": 1e-5}, {"params": vision_params, "lr": 1e-6}, {"params": llm_params, "lr": 2e-6}]
    optimizer = torch.optim.AdamW(groups, lr=2e-6, foreach=True, weight_decay=0.01)

    spec = SyntheticSpec(kind="vlm", seq_len=args.seq_len, vocab_size=t.vocab_size, seed=42)
    # rows are produced and pinned by a background thread, like the reference's loader workers
    # (num_workers=2, reference: train/train_qwen.py:239-250); the timed loop only does the H2D copies
    from vlm_training_b200.data.loader import PrefetchLoader

    data = PrefetchLoader(SyntheticDataset(spec, ours, dp_rank=dp_rank, dp_size=dp_size), depth=3)

    def host_batch():
        b = next(data)
        return {k: b[k] for k in ("input_ids", "labels", "cu_seqlens", "pixel_values", "image_grid_thw")}

    def to_dev(b):
        return {"input_ids": b["input_ids"].to(dev, non_blocking=True).unsqueeze(0),
                "attention_mask": b["cu_seqlens"].to(dev, non_blocking=True),
                "labels": b["labels"].to(dev, non_blocking=True).unsqueeze(0),
                "pixel_values": b["pixel_values"].to(dev, dtype=torch.bfloat16, non_blocking=True),
                "image_grid_thw": b["image_grid_thw"].to(dev, non_blocking=True)}

    def step(batch):
        with torch.autocast("cuda", torch.bfloat16):
            out = model(**batch)
            loss = out.loss
        with torch.autocast("cuda", torch.bfloat16):
            loss.backward()
        optimizer.step()
        optimizer.zero_grad()
        return loss.detach()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        tt = torch.tensor([x], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    try:
        staged = [to_dev(host_batch()) for _ in range(max(2, min(4, args.steps)))]
        if compiled:
            try:  # extra untimed steps so that (re)compilation for the row shapes is over before the warm-up proper
                for i in range(len(staged) + 2):
                    step(staged[i % len(staged)])
            except torch.OutOfMemoryError:
                raise
            except Exception as exc:
                sys.stderr.write(f"[reference harness] torch.compile failed ({type(exc).__name__}: {str(exc)[:200]}); "
                                 "re-running eagerly\n")
                sys.stderr.flush()
                os.environ["REF_COMPILE"] = "0"
                os.environ["REF_COMPILE_FAILED"] = "1"
                os.execv(sys.executable, [sys.executable] + sys.argv)
        for i in range(args.warmup):
            step(staged[i % len(staged)])
        barrier()
        torch.cuda.reset_peak_memory_stats()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            loss = step(staged[i % len(staged)])
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        clocks = sampler.stop() if rank == 0 else None
        peak = torch.cuda.max_memory_allocated() / 2 ** 30
        global_tokens = float(args.seq_len * dp_size)
        value = global_tokens * args.steps / (ms / 1e3)
        e2e = None
        if not args.skip_e2e:
            for _ in range(2):
                step(to_dev(host_batch()))
            barrier()
            h2d = 0
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            for _ in range(args.steps):
                hb = host_batch()
                h2d += sum(hb[k].numel() * hb[k].element_size() for k in hb if torch.is_tensor(hb[k]))
                l = step(to_dev(hb))
                l.item()
            e1.record()
            barrier()
            ms2 = max_over_ranks(e0.elapsed_time(e1))
            e2e = {"value": global_tokens * args.steps / (ms2 / 1e3), "unit": "tokens/s", "ms_per_step": ms2 / args.steps,
                   "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": 4}
    except torch.OutOfMemoryError as exc:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"out of memory with ac_mode={ac_mode}: {str(exc)[:160]}"}))
        dist.destroy_process_group()
        return
    if rank == 0:
        print(json.dumps({
            "metric": "tokens/sec (whole job), Qwen3-VL-8B-shaped VLM training step", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic packed multimodal rows, random-init weights",
            "impl": "reference", "tokens_per_sec_per_gpu": value / world,
            "config": {"model": args.model, "global_batch": dp_size, "seq_len": args.seq_len, "parallelism": f"fsdp{dp_size}xtp{tp}",
                       "ac_mode": ac_mode, "compile": compiled, "optimizer": "torch AdamW foreach on bf16 parameters",
                       "layers_override": args.layers or None,
                       "note": "; ".join(x for x in (note, "torch.compile failed on this box, measured eagerly"
                                                     if os.environ.get("REF_COMPILE_FAILED") == "1" else None) if x) or None},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 0, "peak_mem_gib": peak, "final_loss": float(loss.item())}))
    dist.destroy_process_group()
