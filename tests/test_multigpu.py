"""Multi-GPU checks (2 GPUs of one node, NCCL): tensor parallelism with sequence parallelism against a
single-GPU run, and the one-kernel reduce-scatter+AdamW+all-gather path against the NCCL path.
Each case runs as torchrun child processes; nothing here waits on a flag inside a kernel."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import json, os, sys
sys.path.insert(0, {root!r})
import torch
from vlm_training_b200.config import ConfigManager, Config
from vlm_training_b200.train.trainer import Trainer
cfg = ConfigManager(Config).parse_args(sys.argv[1:])
tr = Trainer(cfg)
hist = tr.train()
with tr.optimizer.all_resident():      # sharded parameters are gathered (a collective: every rank enters)
    # a sample of updated weights: Adam hides a wrong gradient SCALE, but a wrongly weighted sum flips update signs
    probe = torch.cat([p.detach().float().flatten()[:512] for n, p in tr.model.named_parameters()
                       if n.endswith("down_proj.weight") or n.endswith("lm_head.weight") or "merger.linear_fc2.weight" in n])
    torch.cuda.synchronize()
if tr.rank == 0:
    os.makedirs(cfg.training.output_dir, exist_ok=True)
    json.dump([m["train/loss"] for m in hist], open(os.path.join(cfg.training.output_dir, "losses.json"), "w"))
    json.dump(probe.tolist(), open(os.path.join(cfg.training.output_dir, "probe.json"), "w"))
    from vlm_training_b200.parallel.engine import _PendingWeightGather
    json.dump(_PendingWeightGather.RUNS, open(os.path.join(cfg.training.output_dir, "wgather.json"), "w"))
if torch.distributed.is_initialized():
    torch.distributed.destroy_process_group()
"""


def _run(tmp_path, nproc, extra, port, env_extra=None):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    out = tmp_path / f"out_{port}"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script), "--model.model_name", "Qwen3-VL-tiny", "--model.preset", "tiny-qwen3-vl-gpu",
           "--model.train_vit", "true", "--training.output_dir", str(out), "--training.total_steps", "4", "--training.warmup_steps", "0",
           "--training.save_steps", "0", "--training.lr_llm", "1e-3", "--training.lr_mlp", "1e-3", "--training.lr_vit", "1e-3",
           "--training.scheduler_type", "cosine", "--training.data_parallel", "fsdp", "--data.synthetic", "vlm",
           "--data.seq_len", "2048", "--wandb.mode", "disabled"] + extra
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", VLMT_PG_TIMEOUT_S="120")
    env.update(env_extra or {})
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env, cwd=ROOT)
    if res.returncode != 0:
        err = res.stderr
        cut = err.find("Traceback")
        raise AssertionError(res.stdout[-1500:] + err[max(0, cut - 200):cut + 3500])
    _run.last_probe = json.load(open(out / "probe.json"))
    _run.last_wgather = json.load(open(out / "wgather.json"))
    return json.load(open(out / "losses.json"))


def test_tp2_sp_matches_one_gpu(tmp_path):
    one = _run(tmp_path, 1, [], 29701)
    tp2 = _run(tmp_path, 2, ["--training.tp_size", "2", "--training.sequence_parallel", "true", "--training.fused_comm", "false"], 29702)
    assert tp2 == pytest.approx(one, rel=3e-2, abs=3e-2)
    # the same run with the layer collectives and the optimizer step on our own NVLink kernels (plain peer loads)
    p2p = _run(tmp_path, 2, ["--training.tp_size", "2", "--training.sequence_parallel", "true", "--training.fused_comm", "true"], 29705,
               {"VLMT_NO_MULTIMEM": "1"})
    assert p2p == pytest.approx(tp2, rel=2e-2, abs=2e-2)


def test_fused_optimizer_matches_nccl(tmp_path):
    nccl = _run(tmp_path, 2, ["--training.fused_comm", "false"], 29703)
    probe_nccl = torch.tensor(_run.last_probe)
    fused = _run(tmp_path, 2, ["--training.fused_comm", "true"], 29704, {"VLMT_NO_MULTIMEM": "1"})
    probe_fused = torch.tensor(_run.last_probe)
    assert fused == pytest.approx(nccl, rel=2e-3, abs=2e-3)
    assert fused[-1] < fused[0]
    # weights after 4 steps at lr 1e-3: a flipped update sign shows as a ~2e-3 difference
    frac_off = ((probe_fused - probe_nccl).abs() > 5e-4).float().mean().item()
    assert frac_off < 0.02, f"{frac_off:.3f} of the sampled weights differ between the fused and the NCCL optimizer step"


def test_in_place_weight_gradients_match_autograd_accumulation(tmp_path):
    """Data parallel over 2 GPUs with bucketed overlap: weight-gradient GEMMs that add straight into the flat gradient
    buffer (and report the parameter to the bucket logic by hand) against gradients accumulated by autograd."""
    base = _run(tmp_path, 2, ["--training.fused_comm", "true"], 29706, {"VLMT_NO_MULTIMEM": "1", "VLMT_WGRAD_IN_PLACE": "0"})
    probe_base = torch.tensor(_run.last_probe)
    inplace = _run(tmp_path, 2, ["--training.fused_comm", "true"], 29707, {"VLMT_NO_MULTIMEM": "1", "VLMT_WGRAD_IN_PLACE": "1"})
    probe_in = torch.tensor(_run.last_probe)
    assert inplace == pytest.approx(base, rel=2e-3, abs=2e-3)
    frac_off = ((probe_in - probe_base).abs() > 5e-4).float().mean().item()
    assert frac_off < 0.02, f"{frac_off:.3f} of the sampled weights differ"


PRIMITIVES = r"""
import os, sys
sys.path.insert(0, {root!r})
import torch
import torch.distributed as dist
from vlm_training_b200.parallel.mesh import init_distributed
from vlm_training_b200.parallel.p2p import P2PComm
from vlm_training_b200.ops import cuda as cu

rank, world, dev = init_distributed("nccl", "cuda")
comm = P2PComm(dist.group.WORLD, dev, slot_elems=1 << 22)
torch.manual_seed(1234)                      # same stream of numbers on every rank
site = object()
worst = 0.0
for it, (R, K, N) in enumerate([(256, 512, 384), (1024, 1024, 2048), (256, 512, 384), (128, 256, 136), (1024, 1024, 2048)]):
    x_all = (torch.randn(world * R, K, device=dev) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()          # forward layout [out, in]
    w_t = (torch.randn(K, N, device=dev) * 0.05).bfloat16()        # dgrad layout: stored [in, out] = [K, N]
    x_loc = x_all[rank * R:(rank + 1) * R].contiguous()
    comm.begin_microbatch()
    for b_mn, wt in ((False, w), (True, w_t)):
        for use_site in (True, False):
            y, x_full = comm.gemm_all_gather(x_loc, wt, b_mn=b_mn, site=site if use_site else None)
            ref = x_all.float() @ (wt.float() if b_mn else wt.float().t())
            torch.cuda.synchronize()
            assert torch.equal(x_full, x_all), f"gathered rows differ (it {{it}}, b_mn {{b_mn}}, site {{use_site}})"
            err = ((y.float() - ref).abs().max() / ref.abs().max()).item()
            worst = max(worst, err)
            assert err < 2e-2, f"gemm_all_gather: relative error {{err}} (it {{it}}, b_mn {{b_mn}})"
    # GEMM -> reduce-scatter with the same operands: every rank holds a partial product of the full rows
    part = (torch.randn(world * R, K, device=dev) * 0.5 + rank).bfloat16()
    out = comm.gemm_reduce_scatter(part, w)
    gathered = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(gathered, part)
    ref = sum(g.float() @ w.float().t() for g in gathered)[rank * R:(rank + 1) * R]
    torch.cuda.synchronize()
    err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
    assert err < 2e-2, f"gemm_reduce_scatter: relative error {{err}}"
cu.check_status()
from vlm_training_b200.parallel import symm
assert symm.guards_enabled() and len(symm._GUARDED) >= 3
symm.check_guards()                      # every canary band around the peer-visible buffers is intact
label, raw, payload = symm._GUARDED[0]
raw[symm.GUARD_BYTES + payload + 5] = 0  # damage one byte behind a buffer (our own allocation: a legal store)
try:
    symm.check_guards()
    raise SystemExit("a damaged guard band was not reported")
except RuntimeError as exc:
    assert "out-of-bounds store" in str(exc)
print(f"rank {{rank}} PRIMITIVES OK worst {{worst:.2e}}", flush=True)
dist.destroy_process_group()
"""


def test_fused_gemm_collectives_match_torch(tmp_path):
    """The all-gather -> GEMM kernel (own rows from the local source, peers' rows gated by their flags, forward and
    input-gradient layouts, persistent site buffer and ring slot, repeated so slots and buffers are reused) and the
    GEMM -> reduce-scatter kernel against fp32 matmuls of the gathered operands."""
    script = tmp_path / "prims.py"
    script.write_text(PRIMITIVES.format(root=ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29711", str(script)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", VLMT_NO_MULTIMEM="1", VLMT_PG_TIMEOUT_S="120", VLMT_FLAG_WAIT_MS="5000",
               VLMT_DEBUG_GUARDS="1")   # canary bands around every symmetric buffer, checked at the end
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("PRIMITIVES OK") == 2, res.stdout[-2000:]


EP_FUSED = r"""
import os, sys
sys.path.insert(0, {root!r})
import torch
import torch.distributed as dist
from vlm_training_b200 import ops
from vlm_training_b200.parallel.mesh import init_distributed
from vlm_training_b200.parallel.ep import EPContext, EPFused, ep_moe_experts
from vlm_training_b200.ops import cuda as cu

rank, world, dev = init_distributed("nccl", "cuda")
E, H, I, k, T = 16, 256, 128, 4, 1000
torch.manual_seed(0)
gate_up = (torch.randn(E, 2 * I, H, device=dev) * 0.05).bfloat16()
down = (torch.randn(E, H, I, device=dev) * 0.05).bfloat16()
El = E // world
ep_nccl = EPContext(group=dist.group.WORLD, size=world, rank=rank, n_experts=E)
ep_fused = EPContext(group=dist.group.WORLD, size=world, rank=rank, n_experts=E)
ep_fused.fused = EPFused(ep_fused, dev)
for it in range(3):                       # several layers' worth of exchanges through the same buffers
    torch.manual_seed(100 + rank + 10 * it)
    x = torch.randn(T, H, device=dev).bfloat16()
    logits = torch.randn(T, E, device=dev)
    if rank == 1:
        logits[:, :4] += 2.0              # unbalanced: most of rank 1's tokens go to rank 0's experts
    logits[:, E - 1] = -1e9               # one expert without tokens
    w, idx = ops.moe_router(logits, k, True)
    g = torch.randn(T, H, device=dev).bfloat16()
    res = []
    for ep in (ep_nccl, ep_fused):
        xi = x.clone().requires_grad_()
        wi = w.clone().requires_grad_()
        gu = gate_up[rank * El:(rank + 1) * El].clone().requires_grad_()
        dn = down[rank * El:(rank + 1) * El].clone().requires_grad_()
        out = ep_moe_experts(xi, gu, dn, wi, idx, ep)
        out.backward(g)
        torch.cuda.synchronize()
        res.append((out.detach().float(), xi.grad.float(), wi.grad.float(), gu.grad.float(), dn.grad.float()))
    for name, a, b in zip(("out", "dx", "dw_routing", "dgate_up", "ddown"), *res):
        err = ((a - b).abs().max() / (a.abs().max() + 1e-6)).item()
        assert err < 3e-2, f"{{name}}: relative error {{err}} (iteration {{it}})"
cu.check_status()
print(f"rank {{rank}} EP FUSED OK", flush=True)
dist.destroy_process_group()
"""


def test_expert_parallel_peer_store_transport_matches_all_to_all(tmp_path):
    """Expert parallelism on 2 GPUs: dispatch / return by peer stores (device-built plan over all ranks' counts, no host
    read) against the all-to-all transport: outputs and every gradient."""
    script = tmp_path / "ep_fused.py"
    script.write_text(EP_FUSED.format(root=ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29712", str(script)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", VLMT_NO_MULTIMEM="1", VLMT_PG_TIMEOUT_S="120", VLMT_FLAG_WAIT_MS="5000")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("EP FUSED OK") == 2, res.stdout[-2000:]


def test_sharded_parameters_match_whole_parameters_on_gpus(tmp_path):
    """ZeRO-3 residency on 2 GPUs (data parallel): parameters gathered per unit by the own peer-pull kernel from symmetric
    shards (fused_comm on) or by the library all-gather (off), gradients reduce-scattered into shards, against the engine
    that keeps parameters and gradients whole."""
    whole = _run(tmp_path, 2, ["--training.fused_comm", "false"], 29721)
    probe_whole = torch.tensor(_run.last_probe)
    for port, fused in ((29722, "true"), (29723, "false")):
        sharded = _run(tmp_path, 2, ["--training.fused_comm", fused, "--training.reshard_params", "true"], port, {"VLMT_NO_MULTIMEM": "1"})
        assert sharded == pytest.approx(whole, rel=2e-3, abs=2e-3)
        frac_off = ((torch.tensor(_run.last_probe) - probe_whole).abs() > 5e-4).float().mean().item()
        assert frac_off < 0.02, f"{frac_off:.3f} of the sampled weights differ (fused_comm {fused})"
        # with our own gathers the qkv weight of every decoder layer (4 layers x 4 steps) and of the ViT blocks arrives inside
        # its GEMM; with the library all-gather never
        assert (_run.last_wgather["gemm"] >= 16) if fused == "true" else (_run.last_wgather["gemm"] == 0), _run.last_wgather
    plain = _run(tmp_path, 2, ["--training.fused_comm", "true", "--training.reshard_params", "true",
                               "--training.reshard_fuse_first_gemm", "false"], 29724, {"VLMT_NO_MULTIMEM": "1"})
    assert _run.last_wgather["gemm"] == 0
    assert plain == pytest.approx(whole, rel=2e-3, abs=2e-3)


def test_fused_optimizer_with_gradient_clipping_matches_nccl(tmp_path):
    """Clipping at a norm small enough to be active every step: the two-kernel form of the NVLink optimizer step (reduced
    shard + sum of squares, one scalar all-reduce, AdamW + parameter push with the clip factor read on the device) against
    the NCCL path, data parallel and tensor parallel."""
    clip = ["--training.clip_grad", "true", "--training.max_grad_norm", "0.05"]
    for extra, ports in (([], (29731, 29732)), (["--training.tp_size", "2", "--training.sequence_parallel", "true"], (29733, 29734))):
        nccl = _run(tmp_path, 2, clip + extra + ["--training.fused_comm", "false"], ports[0])
        probe_nccl = torch.tensor(_run.last_probe)
        fused = _run(tmp_path, 2, clip + extra + ["--training.fused_comm", "true"], ports[1], {"VLMT_NO_MULTIMEM": "1"})
        assert fused == pytest.approx(nccl, rel=3e-3, abs=3e-3)
        frac_off = ((torch.tensor(_run.last_probe) - probe_nccl).abs() > 5e-4).float().mean().item()
        assert frac_off < 0.02, f"{frac_off:.3f} of the sampled weights differ"
