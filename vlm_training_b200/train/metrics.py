"""Distributed scalar reductions and per-rank performance ranking
(reference: train/utils.py:487-527, train/train_qwen.py:444-476)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _reduce(value: float, op, group, device) -> float:
    if not dist.is_initialized() or (group is None and dist.get_world_size() == 1):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64 if device.type == "cpu" else torch.float32, device=device)
    dist.all_reduce(t, op=op, group=group)
    return float(t.item())


def dist_sum(value, group=None, device=torch.device("cpu")) -> float:
    return _reduce(value, dist.ReduceOp.SUM, group, device)


def dist_max(value, group=None, device=torch.device("cpu")) -> float:
    return _reduce(value, dist.ReduceOp.MAX, group, device)


def dist_mean(value, group=None, device=torch.device("cpu")) -> float:
    if not dist.is_initialized():
        return float(value)
    n = dist.get_world_size(group)
    return _reduce(value, dist.ReduceOp.SUM, group, device) / n


def reduce_many(values: list[float], ops: list[str], group=None, device=torch.device("cpu")) -> list[float]:
    """Several scalars in at most three collectives (one per reduction kind) instead of one each."""
    if not dist.is_initialized():
        return [float(v) for v in values]
    out = list(values)
    n = dist.get_world_size(group)
    for kind, op in (("sum", dist.ReduceOp.SUM), ("mean", dist.ReduceOp.SUM), ("max", dist.ReduceOp.MAX)):
        idx = [i for i, o in enumerate(ops) if o == kind]
        if not idx:
            continue
        t = torch.tensor([float(values[i]) for i in idx], dtype=torch.float32, device=device)
        dist.all_reduce(t, op=op, group=group)
        vals = t.tolist()
        for i, v in zip(idx, vals):
            out[i] = v / n if kind == "mean" else v
    return out


def gather_perf(vector: list[float], device) -> torch.Tensor:
    """All-gather one fp32 vector per rank → ``[world, len(vector)]``."""
    t = torch.tensor(vector, dtype=torch.float32, device=device)
    if not dist.is_initialized():
        return t.unsqueeze(0).cpu()
    out = torch.empty(dist.get_world_size() * t.numel(), dtype=torch.float32, device=device)
    dist.all_gather_into_tensor(out, t)
    return out.view(dist.get_world_size(), t.numel()).cpu()


PERF_KEYS = ("tps", "step_time", "fwd_bwd_time", "tflops", "mfu", "peak_mem_gib")


def topk_report(table: torch.Tensor, k: int) -> dict:
    """K slowest / fastest ranks per metric → ``perf_topk/{metric}_{slow|fast}_{i}[_rank]`` entries."""
    out = {}
    k = min(k, table.shape[0])
    for j, key in enumerate(PERF_KEYS):
        col = table[:, j]
        higher_is_slow = key in ("step_time", "fwd_bwd_time", "peak_mem_gib")
        order = torch.argsort(col, descending=higher_is_slow)
        for i in range(k):
            out[f"perf_topk/{key}_slow_{i}"] = float(col[order[i]])
            out[f"perf_topk/{key}_slow_{i}_rank"] = int(order[i])
            out[f"perf_topk/{key}_fast_{i}"] = float(col[order[-1 - i]])
            out[f"perf_topk/{key}_fast_{i}_rank"] = int(order[-1 - i])
    return out
