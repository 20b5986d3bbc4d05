"""End-to-end trainer on CPU: single process and 2 gloo ranks (FSDP), loss parity between them,
checkpoint save → resume reproducing the uninterrupted loss curve."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg(tmp, **over):
    from vlm_training_b200.config import Config

    cfg = Config()
    cfg.model.model_name, cfg.model.preset = "Qwen3-tiny", "tiny-qwen3"
    t = cfg.training
    t.output_dir, t.bfloat16, t.device = str(tmp), False, "cpu"
    t.data_parallel, t.lr_llm, t.total_steps, t.warmup_steps, t.save_steps = "fsdp", 3e-4, 4, 0, 0
    t.scheduler_type, t.seed = "cosine", 0
    cfg.data.synthetic, cfg.data.seq_len, cfg.data.doc_len_min, cfg.data.doc_len_max = "text-uniform", 256, 16, 128
    cfg.wandb.mode = "disabled"
    for k, v in over.items():
        sec, key = k.split("__")
        setattr(getattr(cfg, sec), key, v)
    return cfg


def _shrink_vocab(monkeypatch):
    # the tiny preset keeps the real 151936-token vocabulary; shrink it so CPU tests stay fast
    from vlm_training_b200.models import config as mc

    orig = mc._PRESETS["tiny-qwen3"]

    def small():
        c = orig()
        c.text.vocab_size = 2048
        return c

    monkeypatch.setitem(mc._PRESETS, "tiny-qwen3", small)


def test_single_process_loss_decreases(tmp_path, monkeypatch):
    _shrink_vocab(monkeypatch)
    from vlm_training_b200.train.trainer import Trainer

    tr = Trainer(_cfg(tmp_path, training__total_steps=8, training__lr_llm=2e-3))
    # uniform-random tokens cannot be learned; train on one fixed row so memorisation shows up in the loss
    fixed = next(tr.loader)
    tr.loader.close()

    class Same:
        def __next__(self):
            return fixed

        def close(self):
            pass

    tr.loader = Same()
    hist = tr.train()
    losses = [m["train/loss"] for m in hist]
    assert len(losses) == 8 and all(l == l for l in losses)
    assert losses[-1] < losses[0]


def test_trainer_reads_rows_from_worker_processes(tmp_path):
    """``data.worker_processes = 2``: the rows come from two spawned processes in a fixed order, so two runs give the same
    loss curve; the workers are gone after ``end_run``."""
    from vlm_training_b200.train.trainer import Trainer

    curves = []
    for run in range(2):
        tr = Trainer(_cfg(tmp_path / f"w{run}", training__total_steps=3, data__worker_processes=2))
        pool = tr.loader.source
        hist = tr.train()
        tr.end_run()
        curves.append([m["train/loss"] for m in hist])
        assert len(hist) == 3 and all(not p.is_alive() for p in pool.procs)
    assert curves[0] == curves[1]


def test_checkpoint_resume_reproduces_curve(tmp_path, monkeypatch):
    _shrink_vocab(monkeypatch)
    from vlm_training_b200.train.trainer import Trainer

    full = Trainer(_cfg(tmp_path / "a", training__total_steps=6)).train()
    first = Trainer(_cfg(tmp_path / "b", training__total_steps=6, training__save_steps=3))
    # stop after 3 steps (as if the job died), then resume in a fresh trainer
    it = first.batch_generator()
    while first.global_step < 3:
        if first.train_step(it) is not None:
            first.may_save()
    first.end_run()
    second = Trainer(_cfg(tmp_path / "b", training__total_steps=6, training__resume_checkpoint=True))
    # the synthetic stream restarts on resume (as the reference's loader does): skip what was consumed
    for _ in range(3):
        next(second.loader)
    hist = second.train()
    assert second.global_step == 6
    a = [m["train/loss"] for m in full[3:]]
    b = [m["train/loss"] for m in hist]
    assert a == pytest.approx(b, rel=1e-5, abs=1e-5)


WORKER = r"""
import json, os, sys
sys.path.insert(0, {root!r})
import torch
from vlm_training_b200.models import config as mc
orig = mc._PRESETS["tiny-qwen3"]
def small():
    c = orig(); c.text.vocab_size = 2048; return c
mc._PRESETS["tiny-qwen3"] = small
from vlm_training_b200.config import ConfigManager, Config
from vlm_training_b200.train.trainer import Trainer
cfg = ConfigManager(Config).parse_args(sys.argv[1:])
tr = Trainer(cfg)
hist = tr.train()
if tr.rank == 0:
    os.makedirs(cfg.training.output_dir, exist_ok=True)
    json.dump([m["train/loss"] for m in hist], open(os.path.join(cfg.training.output_dir, "losses.json"), "w"))
torch.distributed.destroy_process_group() if torch.distributed.is_initialized() else None
"""


def _run_ranks(tmp_path, nproc, extra, port, preset="tiny-qwen3", synthetic="text-uniform", seq_len="256"):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    out = tmp_path / f"out{nproc}"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script),
           "--model.model_name", "Qwen3-VL-tiny" if "vl" in preset else "Qwen3-tiny", "--model.preset", preset,
           "--model.train_vit", "true", "--training.device", "cpu",
           "--training.bfloat16", "false", "--training.output_dir", str(out), "--training.total_steps", "4",
           "--training.warmup_steps", "0", "--training.save_steps", "0", "--training.lr_llm", "3e-4",
           "--training.scheduler_type", "cosine", "--data.synthetic", synthetic, "--data.seq_len", seq_len,
           "--training.lr_mlp", "3e-4", "--training.lr_vit", "3e-4",
           "--data.doc_len_min", "16", "--data.doc_len_max", "128", "--wandb.mode", "disabled"] + extra
    env = dict(os.environ, OMP_NUM_THREADS="2")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return json.load(open(out / "losses.json"))


@pytest.mark.slow
def test_fsdp2_and_ddp2_gloo_agree(tmp_path):
    """FSDP (sharded optimizer) and DDP over 2 gloo ranks see the same data and must give the same losses."""
    fsdp = _run_ranks(tmp_path, 2, ["--training.data_parallel", "fsdp"], 29621)
    ddp = _run_ranks(tmp_path, 2, ["--training.data_parallel", "ddp"], 29622)
    assert fsdp == pytest.approx(ddp, rel=1e-5, abs=1e-5)
    assert fsdp[-1] < fsdp[0] + 0.5


@pytest.mark.slow
def test_tp2_sequence_parallel_matches_single_rank(tmp_path):
    """TP=2 with sequence parallelism computes the same function as one rank (fp32, same data, same init)."""
    one = _run_ranks(tmp_path, 1, [], 29623)
    tp2 = _run_ranks(tmp_path, 2, ["--training.tp_size", "2", "--training.sequence_parallel", "true"], 29624)
    tp2_nosp = _run_ranks(tmp_path, 2, ["--training.tp_size", "2"], 29625)
    assert tp2 == pytest.approx(one, rel=2e-4, abs=2e-4)
    assert tp2_nosp == pytest.approx(one, rel=2e-4, abs=2e-4)


@pytest.mark.slow
def test_vlm_tp2_image_parallel_vit_matches_single_rank(tmp_path):
    """Under TP the vision tower runs image-parallel and its features are exchanged; with and without sequence
    parallelism the losses must follow the single-rank run (fp32, gloo)."""
    kw = dict(preset="tiny-qwen3-vl-gpu", synthetic="vlm", seq_len="1024")
    one = _run_ranks(tmp_path, 1, [], 29626, **kw)
    sp = _run_ranks(tmp_path, 2, ["--training.tp_size", "2", "--training.sequence_parallel", "true"], 29627, **kw)
    nosp = _run_ranks(tmp_path, 2, ["--training.tp_size", "2"], 29628, **kw)
    assert sp == pytest.approx(one, rel=5e-4, abs=5e-4)
    assert nosp == pytest.approx(one, rel=5e-4, abs=5e-4)


@pytest.mark.slow
def test_vlm_dp2_tp2_matches_dp2(tmp_path):
    """Four ranks as data-parallel 2 x tensor-parallel 2 (two reduction domains in the optimizer engine: parameters split
    over TP are reduced over the data-parallel group, replicated ones over the world) follow the 2-rank data-parallel run."""
    kw = dict(preset="tiny-qwen3-vl-gpu", synthetic="vlm", seq_len="1024")
    dp2 = _run_ranks(tmp_path, 2, ["--training.data_parallel", "fsdp"], 29629, **kw)
    dp2tp2 = _run_ranks(tmp_path, 4, ["--training.data_parallel", "fsdp", "--training.tp_size", "2",
                                      "--training.sequence_parallel", "true"], 29630, **kw)
    assert dp2tp2 == pytest.approx(dp2, rel=5e-4, abs=5e-4)


@pytest.mark.slow
@pytest.mark.parametrize("ac", ["off", "full"])
def test_sharded_parameters_match_whole_parameters(tmp_path, ac):
    """ZeRO-3 residency (parameters and gradients sharded; a layer's parameters gathered for its forward / recomputation /
    backward and released afterwards; gradients reduce-scattered per micro-batch) against the engine that keeps them whole:
    same losses on 2 gloo ranks, with and without activation checkpointing, with gradient accumulation."""
    common = ["--training.data_parallel", "fsdp", "--training.ac_mode", ac, "--training.tpi_multiplier", "1.5"]
    whole = _run_ranks(tmp_path, 2, common, 29631)
    sharded = _run_ranks(tmp_path, 2, common + ["--training.reshard_params", "true"], 29632)
    assert sharded == pytest.approx(whole, rel=1e-5, abs=1e-5)
    keep = _run_ranks(tmp_path, 2, common + ["--training.reshard_params", "true", "--training.reshard_after_forward", "false"], 29633)
    assert keep == pytest.approx(whole, rel=1e-5, abs=1e-5)


@pytest.mark.slow
def test_sharded_parameters_under_dp2_tp2_and_checkpoint_resume(tmp_path):
    """Sharded parameters with two reduction domains (dp 2 x tp 2, VLM with image-parallel ViT), and a checkpoint written
    and resumed with parameters sharded."""
    kw = dict(preset="tiny-qwen3-vl-gpu", synthetic="vlm", seq_len="1024")
    tp = ["--training.data_parallel", "fsdp", "--training.tp_size", "2", "--training.sequence_parallel", "true"]
    whole = _run_ranks(tmp_path, 4, tp, 29634, **kw)
    sharded = _run_ranks(tmp_path, 4, tp + ["--training.reshard_params", "true"], 29635, **kw)
    assert sharded == pytest.approx(whole, rel=5e-5, abs=5e-5)
    # 2 steps and a checkpoint, then a fresh job resumes from it (parameters are gathered for the state dict and
    # re-sharded after the load)
    base = ["--training.data_parallel", "fsdp", "--training.reshard_params", "true"]
    (tmp_path / "full").mkdir()
    (tmp_path / "part").mkdir()
    full = _run_ranks(tmp_path / "full", 2, base, 29636)
    first = _run_ranks(tmp_path / "part", 2, base + ["--training.total_steps", "2", "--training.save_steps", "2"], 29637)
    assert first == pytest.approx(full[:2], rel=1e-6, abs=1e-6)
    assert os.path.exists(tmp_path / "part" / "out2" / "checkpoint-step-2" / ".metadata")
    rest = _run_ranks(tmp_path / "part", 2, base + ["--training.resume_checkpoint", "true"], 29638)
    assert len(rest) == 2 and all(l == l and l < 20 for l in rest)
