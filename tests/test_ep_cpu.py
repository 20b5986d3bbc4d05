"""Expert parallelism on two gloo ranks: the all-to-all dispatch/combine path must give the same outputs and
gradients as running every expert locally, and training with it must follow the same loss curve."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import torch
import torch.distributed as dist
from vlm_training_b200 import ops
from vlm_training_b200.parallel.ep import EPContext, ep_moe_experts

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(0)
E, H, I, k = 8, 32, 16, 2
gate_up = torch.randn(E, 2 * I, H) * 0.2
down = torch.randn(E, H, I) * 0.2
torch.manual_seed(100 + rank)
T = 37 + 5 * rank                      # different token counts per rank
x = torch.randn(T, H, requires_grad=True)
logits = torch.randn(T, E)
if rank == 1:
    logits[:, :4] += 3.0               # unbalanced routing: most of rank 1's tokens go to rank 0's experts
w, idx = ops.moe_router(logits, k, True)
g = torch.randn(T, H)

# every expert local
gu_full, dn_full = gate_up.clone().requires_grad_(), down.clone().requires_grad_()
want = ops.moe_experts(x, gu_full, dn_full, w, idx)
want.backward(g)
dx_want = x.grad.clone(); x.grad = None
dist.all_reduce(gu_full.grad); dist.all_reduce(dn_full.grad)

# expert parallel
ep = EPContext(group=dist.group.WORLD, size=world, rank=rank, n_experts=E)
El = E // world
gu_loc = gate_up[rank * El:(rank + 1) * El].clone().requires_grad_()
dn_loc = down[rank * El:(rank + 1) * El].clone().requires_grad_()
got = ep_moe_experts(x, gu_loc, dn_loc, w, idx, ep)
got.backward(g)
torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
torch.testing.assert_close(x.grad, dx_want, atol=1e-5, rtol=1e-5)
torch.testing.assert_close(gu_loc.grad, gu_full.grad[rank * El:(rank + 1) * El], atol=1e-5, rtol=1e-5)
torch.testing.assert_close(dn_loc.grad, dn_full.grad[rank * El:(rank + 1) * El], atol=1e-5, rtol=1e-5)
print(f"rank {rank} ok", flush=True)
dist.destroy_process_group()
'''

TRAIN_WORKER = r'''
import json, os, sys
import torch
from vlm_training_b200.config import ConfigManager
from vlm_training_b200.train.trainer import Trainer

out = sys.argv[1]
ep = int(sys.argv[2])
cfg = ConfigManager().parse_args(["--model.preset", "tiny-qwen3.5-moe", "--training.random_init", "true",
    "--training.output_dir", out, "--training.total_steps", "3", "--training.warmup_steps", "1", "--training.device", "cpu",
    "--training.ep_size", str(ep), "--training.data_parallel", "fsdp", "--training.save_steps", "3",
    "--data.synthetic", "text-uniform", "--data.seq_len", "128", "--data.doc_len_min", "16", "--data.doc_len_max", "64",
    "--wandb.mode", "disabled"])
tr = Trainer(cfg)
losses = tr.train()
if int(os.environ.get("RANK", "0")) == 0:
    json.dump({"losses": [float(l["train/loss"]) for l in losses]}, open(os.path.join(out, f"ep{ep}.json"), "w"))
'''


def _run(tmp_path, script, args, port, nproc=2):
    path = tmp_path / "worker.py"
    path.write_text(script)
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(path)] + args
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res


def test_ep2_dispatch_combine_matches_local_experts(tmp_path):
    res = _run(tmp_path, WORKER, [], 29631)
    assert "rank 0 ok" in res.stdout and "rank 1 ok" in res.stdout


def test_ep2_training_matches_ep1(tmp_path):
    """Same data, same init: two data-parallel ranks with and without expert parallelism follow the same loss curve."""
    import json

    a, b = tmp_path / "ep1", tmp_path / "ep2"
    a.mkdir(); b.mkdir()
    _run(tmp_path, TRAIN_WORKER, [str(a), "1"], 29632)
    _run(tmp_path, TRAIN_WORKER, [str(b), "2"], 29633)
    la = json.load(open(a / "ep1.json"))["losses"]
    lb = json.load(open(b / "ep2.json"))["losses"]
    assert len(la) == len(lb) == 3
    for x, y in zip(la, lb):
        assert abs(x - y) < 2e-3 * max(1.0, abs(x)), (la, lb)
