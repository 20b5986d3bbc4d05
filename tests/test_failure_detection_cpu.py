"""Failure detection without a device fault: every failure is made on the host (a rank that leaves, a data worker
that raises, a checkpoint that is incomplete) and must surface as a Python exception in bounded time."""
import os
import subprocess
import sys
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LOST_RANK = r'''
import os, sys, time
import torch
import torch.distributed as dist
from vlm_training_b200.parallel.mesh import init_distributed

rank, world, dev = init_distributed(backend="gloo", device="cpu")
x = torch.ones(4)
dist.all_reduce(x)                      # step 1: everybody is there
assert float(x[0]) == world
if rank == 1:
    # leaves between steps, with nothing in flight
    dist.destroy_process_group()
    sys.exit(0)
t0 = time.time()
try:
    for _ in range(3):                  # the survivors' next collectives must end with an error, not hang
        dist.all_reduce(x)
    print("NOT DETECTED", flush=True)
    sys.exit(3)
except Exception as exc:
    print(f"rank {rank} DETECTED after {time.time() - t0:.1f}s: {type(exc).__name__}", flush=True)
    sys.exit(0)
'''


def test_lost_rank_ends_next_collective_with_error(tmp_path):
    """A rank that leaves between steps: the others' next collective raises within the (short) process-group
    timeout instead of waiting forever."""
    path = tmp_path / "lost.py"
    path.write_text(LOST_RANK)
    env = dict(os.environ, PYTHONPATH=ROOT, VLMT_PG_TIMEOUT_S="10", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29651", str(path)]
    t0 = time.time()
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=env, cwd=ROOT)
    assert time.time() - t0 < 120
    out = res.stdout + res.stderr
    assert "NOT DETECTED" not in out, out[-2000:]
    assert out.count("DETECTED after") == 2, out[-2000:]


def test_data_worker_exception_reaches_the_training_thread():
    from vlm_training_b200.data.loader import PrefetchLoader

    class Boom:
        def __init__(self):
            self.n = 0

        def __iter__(self):
            return self

        def __next__(self):
            self.n += 1
            if self.n == 3:
                raise ValueError("bad sample 3")
            ids = torch.arange(8)
            return {"input_ids": ids, "labels": ids.clone(), "cu_seqlens": torch.tensor([0, 8], dtype=torch.int32)}

    loader = PrefetchLoader(Boom(), depth=2, pin=False)
    next(loader)
    next(loader)
    with pytest.raises(ValueError, match="bad sample 3"):
        next(loader)
    loader.close()


def test_incomplete_checkpoint_is_refused(tmp_path):
    """A checkpoint directory without its metadata file (a save that was interrupted) is not a resume point."""
    from vlm_training_b200.train import checkpoint as ckpt

    d = tmp_path / "checkpoint-step-7"
    d.mkdir()
    (d / "__0_0.distcp").write_bytes(b"\0" * 16)
    assert ckpt.latest_step(str(tmp_path)) in (None, 7)
    with pytest.raises(FileNotFoundError):
        ckpt.load_checkpoint(str(tmp_path), 7, model=None, engine=None, scheduler=None)


def test_device_status_word_raises_on_host():
    """The kernels report a wait that ran out through a status word; the host check turns a non-zero word into an
    exception and clears it (exercised here on a fake status tensor, no GPU involved)."""
    from vlm_training_b200.ops import status

    word = torch.zeros(1, dtype=torch.int32)
    status.raise_if_set(word, "test kernel")          # zero: nothing happens
    word[0] = 3
    with pytest.raises(RuntimeError, match="test kernel.*TMEM"):
        status.raise_if_set(word, "test kernel")
    assert int(word[0]) == 0


# ----------------------------------------------------------------------------- data worker processes
def _pool_args(tmp_path, synthetic="text-uniform", data_path=""):
    from vlm_training_b200.config import Config
    from vlm_training_b200.models.config import ModelConfig

    cfg = Config()
    cfg.data.synthetic = synthetic
    cfg.data.seq_len = 256
    cfg.data.doc_len_min, cfg.data.doc_len_max = 16, 64
    cfg.data.data_path = data_path
    cfg.training.seed = 3
    return (cfg.data, cfg.training, ModelConfig.preset("tiny-qwen3"), 0, 1)


def test_worker_processes_deliver_rows_in_a_fixed_order(tmp_path):
    """Two worker processes, rows taken in round-robin order: two pools give the same sequence, and it interleaves the two
    workers' own streams."""
    from vlm_training_b200.data.loader import WorkerPool, make_dataset

    args = _pool_args(tmp_path)
    seqs = []
    for _ in range(2):
        pool = WorkerPool(args, 2, depth=2)
        try:
            seqs.append([next(pool)["input_ids"].clone() for _ in range(6)])
        finally:
            pool.close()
    for a, b in zip(*seqs):
        assert torch.equal(a, b)
    w0 = iter(make_dataset(*args, worker=(0, 2)))
    w1 = iter(make_dataset(*args, worker=(1, 2)))
    want = [next(w0 if i % 2 == 0 else w1)["input_ids"] for i in range(6)]
    for a, b in zip(seqs[0], want):
        assert torch.equal(a, b)
    assert not torch.equal(seqs[0][0], seqs[0][1])


def test_a_failing_data_worker_process_is_reported_in_the_training_process(tmp_path):
    """A worker that cannot build its dataset (a data path that does not exist) raises here, with the worker's traceback."""
    from vlm_training_b200.data.loader import WorkerPool

    args = _pool_args(tmp_path, synthetic="no-such-kind")
    pool = WorkerPool(args, 2, depth=2)
    try:
        with pytest.raises(RuntimeError, match="data worker [01] failed: ValueError"):
            next(pool)
    finally:
        pool.close()


def test_a_data_worker_process_that_dies_silently_is_noticed(tmp_path):
    """The worker is killed by the test between two rows (a host-side failure: nothing runs on a GPU); the next read
    that finds its queue empty reports the exit code instead of waiting for ever."""
    from vlm_training_b200.data.loader import WorkerPool

    pool = WorkerPool(_pool_args(tmp_path), 2, depth=1)
    try:
        next(pool)
        pool.procs[1].kill()
        pool.procs[1].join(timeout=10)
        with pytest.raises(RuntimeError, match="data worker 1 exited with code"):
            for _ in range(8):       # rows already queued by the dead worker may still arrive first
                next(pool)
    finally:
        pool.close()
