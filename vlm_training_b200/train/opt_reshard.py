"""Loading an optimizer checkpoint under a different parallel layout.

The engine's optimizer state (fp32 master weights and both Adam moments) is saved as it lives in memory: one flat
tensor per bucket and reduction domain, sharded over the domain's ranks, one set per tensor-parallel and per
expert-parallel rank (:mod:`.checkpoint`).  That loads back in place when the layout is unchanged.  A run that
resumes with another ``tp_size``, ``ep_size``, data-parallel size or bucket size cannot use those tensors
directly, so every checkpoint also carries ``optimizer_layout.json``: for every domain the bucket boundaries and,
per parameter, its name, offset, local shape and how it is split over tensor-parallel ranks.  With it the state is
re-assembled parameter by parameter:

    old bucket shards --DCP--> whole old bucket (host memory, one bucket at a time)
      --slice--> the parameter's piece of every old tensor-parallel / expert-parallel rank
      --concatenate--> the GLOBAL state tensor of the parameter
      --split for the new tensor-parallel / expert-parallel rank--> flat --> this rank's shard of the new bucket

The reference gets the same ability from DTensor placements (reference: train/train_qwen.py:338-352); here the
buckets are flat, so the bookkeeping is explicit.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

LAYOUT_FILE = "optimizer_layout.json"
STATE_NAMES = ("master", "exp_avg", "exp_avg_sq")


def _param_names(model) -> dict:
    return {p: n for n, p in model.named_parameters()}


def describe_layout(engine, tp_size: int = 1) -> dict:
    """JSON-serialisable description of where every parameter's optimizer state lives in this engine."""
    names = _param_names(engine.model)
    ep = getattr(engine.model, "_ep_ctx", None)
    out = {"version": 1, "tp_size": int(tp_size), "ep_size": int(ep.size) if ep is not None else 1, "domains": {}}
    for d in engine.domains:
        params = []
        for p, off, n, _gi in d.slots:
            params.append({"name": names[p], "offset": int(off), "numel": int(n), "shape": list(p.shape),
                           "tp_dim": getattr(p, "_tp_shard_dim", None) if getattr(p, "_tp_sharded", False) else None,
                           "tp_splits": list(getattr(p, "_tp_splits", None) or []) if getattr(p, "_tp_sharded", False) else None,
                           "ep": bool(getattr(p, "_ep_sharded", False))})
        out["domains"][d.name] = {"size": int(d.size), "shard": bool(d.shard), "total": int(d.total),
                                  "buckets": [[int(b.start), int(b.end)] for b in d.buckets],
                                  "state_dtype": str(d.exp_avg[0].dtype).replace("torch.", "") if d.exp_avg else "float32",
                                  "params": params}
    return out


def write_layout(path: str, engine, tp_size: int = 1):
    if not dist.is_initialized() or dist.get_rank() == 0:
        with open(os.path.join(path, LAYOUT_FILE), "w") as fh:
            json.dump(describe_layout(engine, tp_size), fh)


def read_layout(path: str) -> dict | None:
    f = os.path.join(path, LAYOUT_FILE)
    if not os.path.exists(f):
        return None
    with open(f) as fh:
        return json.load(fh)


def same_layout(a: dict, b: dict) -> bool:
    return json.dumps(a, sort_keys=True) == json.dumps(b, sort_keys=True)


# ----------------------------------------------------------------------------- tensor-parallel split / concatenate (local maths)
def tp_concat(pieces: list[torch.Tensor], dim: int, splits: list[int]) -> torch.Tensor:
    """Inverse of the per-split sharding of ``parallel.tp``: ``pieces[r]`` holds rank r's 1/tp of every split."""
    tp = len(pieces)
    if tp == 1:
        return pieces[0]
    if dim == 1:
        return torch.cat(pieces, 1)
    per_rank = [n // tp for n in splits]
    out = []
    for si in range(len(splits)):
        o = sum(per_rank[:si])
        for r in range(tp):
            out.append(pieces[r].narrow(0, o, per_rank[si]))
    return torch.cat(out, 0)


def tp_take(full: torch.Tensor, dim: int, splits: list[int], tp: int, rank: int) -> torch.Tensor:
    if tp == 1:
        return full
    if dim == 1:
        n = full.shape[1] // tp
        return full.narrow(1, rank * n, n)
    out, o = [], 0
    for n in splits:
        k = n // tp
        out.append(full.narrow(0, o + rank * k, k))
        o += n
    return torch.cat(out, 0)


def _prefixes(domain_name: str, layout: dict) -> list[str]:
    """Checkpoint key prefixes that hold one saved domain (one per tensor-parallel / expert-parallel rank)."""
    if domain_name == "tp_sharded":
        return [f"tp_sharded.tp{r}" for r in range(layout["tp_size"])]
    if domain_name == "ep_experts":
        return [f"ep_experts.ep{r}" for r in range(layout["ep_size"])]
    return [domain_name]


def load_resharded(path: str, engine, saved: dict, tp_ctx=None):
    """Fill ``engine``'s master weights and moments from a checkpoint written under the layout ``saved``."""
    import torch.distributed.checkpoint as dcp

    names = _param_names(engine.model)
    ep = getattr(engine.model, "_ep_ctx", None)
    new_tp = tp_ctx.size if (tp_ctx is not None and tp_ctx.enabled) else 1
    new_tp_rank = tp_ctx.rank if new_tp > 1 else 0
    new_ep = ep.size if ep is not None else 1
    new_ep_rank = ep.rank if ep is not None else 0
    # where every parameter goes in the new engine
    target = {}
    for d in engine.domains:
        for p, off, n, _gi in d.slots:
            target[names[p]] = (d, p, off, n)
    filled = set()
    no_dist = not dist.is_initialized()
    dtype_of = {"float32": torch.float32, "bfloat16": torch.bfloat16}
    for dname, dom in saved["domains"].items():
        prefixes = _prefixes(dname, saved)
        sdt = dtype_of[dom["state_dtype"]]
        for bi, (bstart, bend) in enumerate(dom["buckets"]):
            # the whole old bucket of every old tensor-parallel / expert-parallel rank, in host memory
            bufs = {pre: {s: torch.empty(bend - bstart, dtype=torch.float32 if s == "master" else sdt) for s in STATE_NAMES}
                    for pre in prefixes}
            request = {"optimizer": {pre: {f"{s}.{bi}": t for s, t in st.items()} for pre, st in bufs.items()}}
            dcp.load(request, checkpoint_id=path, no_dist=no_dist)
            for ent in dom["params"]:
                if not (bstart <= ent["offset"] < bend):
                    continue
                tgt = target.get(ent["name"])
                if tgt is None:
                    continue  # a parameter that is frozen (or absent) in this run
                d, p, off, n = tgt
                lo_old = ent["offset"] - bstart
                for s in STATE_NAMES:
                    pieces = [bufs[pre][s][lo_old:lo_old + ent["numel"]].view(ent["shape"]) for pre in prefixes]
                    if ent["ep"]:
                        full = torch.cat(pieces, 0) if len(pieces) > 1 else pieces[0]
                    elif ent["tp_dim"] is not None:
                        full = tp_concat(pieces, ent["tp_dim"], ent["tp_splits"])
                    else:
                        full = pieces[0]
                    # the new rank's part of the global tensor
                    if getattr(p, "_ep_sharded", False):
                        k = full.shape[0] // new_ep
                        local = full.narrow(0, new_ep_rank * k, k)
                    elif getattr(p, "_tp_sharded", False):
                        local = tp_take(full, p._tp_shard_dim, list(p._tp_splits), new_tp, new_tp_rank)
                    else:
                        local = full
                    if local.numel() != n:
                        raise ValueError(f"optimizer state of {ent['name']}: {tuple(local.shape)} does not match the parameter "
                                         f"{tuple(p.shape)} of this run")
                    flat = local.reshape(-1)
                    dst_list = {"master": d.master, "exp_avg": d.exp_avg, "exp_avg_sq": d.exp_avg_sq}[s]
                    for nbi, nb in enumerate(d.buckets):
                        slo, shi = d.shard_range(nb)
                        a, b = max(off, slo), min(off + n, shi)
                        if b > a:
                            dst = dst_list[nbi]
                            dst[a - slo:b - slo].copy_(flat[a - off:b - off].to(dst.dtype))
                filled.add(ent["name"])
    missing = sorted(set(target) - filled)
    if missing:
        raise KeyError(f"the checkpoint holds no optimizer state for {missing[:5]}{' ...' if len(missing) > 5 else ''}")
