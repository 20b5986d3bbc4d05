"""An optimizer checkpoint written under one parallel layout loads under another: data-parallel 2 -> tensor-parallel 2 ->
one process with other bucket sizes.  The state is made recognisable (first moment = master / 2, second moment =
master squared, master = the seeded initial weights), so after a resharded load every element can be checked."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import torch
from vlm_training_b200.models import config as mc
orig = mc._PRESETS["tiny-qwen3.5"]
mc._PRESETS["tiny-qwen3.5"] = orig
from vlm_training_b200.config import ConfigManager, Config
from vlm_training_b200.train.trainer import Trainer
import vlm_training_b200.parallel.engine as eng

phase, bucket_mb = os.environ["PHASE"], float(os.environ.get("BUCKET_MB", "256"))
_init = eng.ShardedOptimizerEngine.__init__
def patched(self, *a, **k):
    k["bucket_mb"] = bucket_mb
    _init(self, *a, **k)
eng.ShardedOptimizerEngine.__init__ = patched
cfg = ConfigManager(Config).parse_args(sys.argv[1:])
tr = Trainer(cfg)
e = tr.optimizer
if phase == "save":
    for d in e.domains:
        for bi in range(len(d.buckets)):
            d.exp_avg[bi].copy_(0.5 * d.master[bi])
            d.exp_avg_sq[bi].copy_(d.master[bi] ** 2)
    e.step_count = 7
    tr.global_step = 1
    tr.save_checkpoint()
else:
    before = [[m.clone() for m in d.master] for d in e.domains]
    for d in e.domains:                    # poison: everything must come from the checkpoint
        for bi in range(len(d.buckets)):
            d.master[bi].fill_(123.0); d.exp_avg[bi].fill_(-7.0); d.exp_avg_sq[bi].fill_(-7.0)
    tr.load_checkpoint(1)
    assert e.step_count == 7
    n = 0
    for di, d in enumerate(e.domains):
        for bi, b in enumerate(d.buckets):
            lo, hi = d.shard_range(b)
            live = torch.zeros(hi - lo, dtype=torch.bool)      # alignment padding between parameters holds no state
            for p, off, cnt, _ in d.slots:
                a, z = max(off, lo), min(off + cnt, hi)
                if z > a:
                    live[a - lo:z - lo] = True
            m = d.master[bi][live]
            assert torch.equal(m, before[di][bi][live]), f"master of {{d.name}} bucket {{bi}} differs from the seeded weights"
            assert torch.allclose(d.exp_avg[bi][live], 0.5 * m), f"first moment of {{d.name}} bucket {{bi}}"
            assert torch.allclose(d.exp_avg_sq[bi][live], m ** 2), f"second moment of {{d.name}} bucket {{bi}}"
            n += int(live.sum())
    print(f"rank {{tr.rank}} RESHARD OK {{n}} elements", flush=True)
    if os.environ.get("RESAVE") == "1":
        tr.global_step = 2
        tr.save_checkpoint()
tr.end_run()
torch.distributed.destroy_process_group() if torch.distributed.is_initialized() else None
"""


def _run(tmp_path, nproc, extra, port, env):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    base = ["--model.model_name", "Qwen3.5-tiny", "--model.preset", "tiny-qwen3.5", "--training.device", "cpu", "--training.bfloat16", "false",
            "--training.output_dir", str(tmp_path / "ckpt"), "--training.total_steps", "4", "--training.save_steps", "0",
            "--training.data_parallel", "fsdp", "--data.synthetic", "text-uniform", "--data.seq_len", "256", "--wandb.mode", "disabled"]
    if nproc == 1:
        cmd = [sys.executable, str(script)] + base + extra
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), str(script)] + base + extra
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2", **env), cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


@pytest.mark.slow
def test_optimizer_state_survives_a_change_of_layout(tmp_path):
    # written by 2 data-parallel ranks with small buckets (several buckets, parameters straddling shard boundaries)
    _run(tmp_path, 2, [], 29641, {"PHASE": "save", "BUCKET_MB": "0.25"})
    assert os.path.exists(tmp_path / "ckpt" / "checkpoint-step-1" / "optimizer_layout.json")
    # read by 2 tensor-parallel ranks (head-split fused projections, Gated-DeltaNet splits) with one big bucket; saved again
    out = _run(tmp_path, 2, ["--training.tp_size", "2", "--training.sequence_parallel", "true"], 29642,
               {"PHASE": "load", "RESAVE": "1"})
    assert out.count("RESHARD OK") == 2
    # the tensor-parallel checkpoint read back by a single process with yet another bucket size
    import shutil

    shutil.rmtree(tmp_path / "ckpt" / "checkpoint-step-1")
    os.rename(tmp_path / "ckpt" / "checkpoint-step-2", tmp_path / "ckpt" / "checkpoint-step-1")
    out = _run(tmp_path, 1, [], 0, {"PHASE": "load", "BUCKET_MB": "0.1"})
    assert out.count("RESHARD OK") == 1
