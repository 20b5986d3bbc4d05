"""Distributed checkpoints in the torch DCP directory format.

Layout and contents follow the reference trainer (reference: train/train_qwen.py:330-401,
621-639): ``<output_dir>/checkpoint-step-<N>/`` holding ``.metadata`` and
``__<rank>_<i>.distcp`` files with the entries ``model`` (HF-style keys, e.g.
``model.model.language_model.layers.0.self_attn.q_proj.weight``), ``optimizer``,
``scheduler``, ``step``, ``tokens_seen`` and ``tokens_seen_assistant``.

* ``model`` tensors are saved as GLOBAL tensors: tensor-parallel shards are gathered at
  save time and re-split at load time, so a checkpoint loads under any (dp, tp).
* ``optimizer`` holds the sharded fp32 master weights and Adam moments, one DTensor per
  bucket (``Shard(0)`` over the reduction group).  ``optimizer_layout.json`` beside them
  records where every parameter's state sits; a run with the same layout loads the shards
  in place, a run with another ``tp_size`` / ``ep_size`` / data-parallel size / bucket size
  re-assembles the state parameter by parameter (:mod:`.opt_reshard`).
* Unlike the reference, a failed save or load raises instead of being logged and ignored.
"""
from __future__ import annotations

import os
import re

import torch
import torch.distributed as dist

from .logger import logger

CKPT_RE = re.compile(r"checkpoint-step-(\d+)$")


def checkpoint_dir(output_dir: str, step: int) -> str:
    return os.path.join(output_dir, f"checkpoint-step-{step}")


def latest_step(output_dir: str) -> int | None:
    """Largest ``N`` among ``checkpoint-step-N`` entries that finished writing (have ``.metadata``)."""
    if not os.path.isdir(output_dir):
        return None
    steps = []
    for name in os.listdir(output_dir):
        m = CKPT_RE.search(name)
        if m and os.path.exists(os.path.join(output_dir, name, ".metadata")):
            steps.append(int(m.group(1)))
    return max(steps) if steps else None


# ----------------------------------------------------------------------------- tensor-parallel gather / split
def _tp_gather(local: torch.Tensor, dim: int, splits: list[int], ctx) -> torch.Tensor:
    """Inverse of the per-split row/column sharding done by ``apply_tp``."""
    parts = [torch.empty_like(local) for _ in range(ctx.size)]
    dist.all_gather(parts, local.contiguous(), group=ctx.group)
    if dim == 1:
        return torch.cat(parts, 1)
    per_rank = [n // ctx.size for n in splits]
    out = []
    for si in range(len(splits)):
        o = sum(per_rank[:si])
        for r in range(ctx.size):
            out.append(parts[r].narrow(0, o, per_rank[si]))
    return torch.cat(out, 0)


def _tp_split(full: torch.Tensor, dim: int, splits: list[int], ctx) -> torch.Tensor:
    if dim == 1:
        n = full.shape[1] // ctx.size
        return full.narrow(1, ctx.rank * n, n)
    out, o = [], 0
    for n in splits:
        k = n // ctx.size
        out.append(full.narrow(0, o + ctx.rank * k, k))
        o += n
    return torch.cat(out, 0)


def _param_meta(model) -> dict:
    """state-dict key → (shard dim, splits) for tensor-parallel sharded entries.  Fused parameters appear
    under their HF names; each HF view inherits the fused parameter's shard dim with its own single split."""
    meta = {}
    tp = getattr(model, "tp", None)
    if tp is None or not tp.enabled:
        return meta
    from ..models.layers import FusedLinear

    fused_children = {}
    for mname, mod in model.named_modules():
        if isinstance(mod, FusedLinear):
            parent = mname.rsplit(".", 1)[0] if "." in mname else ""
            for split_name in mod.splits:
                fused_children[f"{parent}.{split_name}.weight" if parent else f"{split_name}.weight"] = (mname, split_name)
    for name, p in model.named_parameters():
        if getattr(p, "_tp_sharded", False):
            meta[name] = (p._tp_shard_dim, p._tp_splits)
    for hf_key, (mname, split_name) in fused_children.items():
        p = model.get_submodule(mname).weight
        if getattr(p, "_tp_sharded", False):
            if split_name == "in_proj_qkv":  # three head-aligned parts inside one HF tensor
                g = model.get_submodule(mname.rsplit(".", 1)[0])
                meta[hf_key] = (0, [g.key_dim * tp.size, g.key_dim * tp.size, g.value_dim * tp.size])
            else:
                meta[hf_key] = (0, None)
    return meta


def model_state_for_save(model) -> dict:
    """HF-keyed state dict of GLOBAL tensors (gathers tensor-parallel shards)."""
    state = model.state_dict()
    tp = getattr(model, "tp", None)
    if tp is None or not tp.enabled:
        return state
    meta = _param_meta(model)
    out = {}
    for k, v in state.items():
        if k in meta:
            dim, splits = meta[k]
            splits = splits if splits is not None else [v.shape[0] * tp.size]
            out[k] = _tp_gather(v, dim, splits, tp)
        else:
            out[k] = v
    return out


def load_model_state(model, state: dict):
    """Copy global tensors into the (possibly tensor-parallel sharded) model, in place."""
    tp = getattr(model, "tp", None)
    target = model.state_dict()
    meta = _param_meta(model) if tp is not None and tp.enabled else {}
    ep = getattr(model, "_ep_ctx", None)
    ep_keys = {}
    if ep is not None and ep.size > 1:  # expert-parallel parameters: state_dict() shows gathered copies, not the parameters
        ep_keys = {n: p for n, p in model.named_parameters() if getattr(p, "_ep_sharded", False)}
    with torch.no_grad():
        for k, p in ep_keys.items():
            n = ep.local_experts
            p.copy_(state[k][ep.rank * n:(ep.rank + 1) * n].to(p.dtype))
        for k, dst in target.items():
            if k in ep_keys:
                continue
            src = state[k]
            if k in meta:
                dim, splits = meta[k]
                splits = splits if splits is not None else [src.shape[0]]
                src = _tp_split(src, dim, splits, tp)
            dst.copy_(src.to(dst.dtype))


def _global_shapes(model) -> dict:
    tp = getattr(model, "tp", None)
    meta = _param_meta(model) if tp is not None and tp.enabled else {}
    shapes = {}
    for k, v in model.state_dict().items():
        shape = list(v.shape)
        if k in meta:
            shape[meta[k][0]] *= tp.size
        shapes[k] = (tuple(shape), v.dtype)
    return shapes


# ----------------------------------------------------------------------------- optimizer <-> DTensor
_MESH_CACHE = {}


def _mesh_for(domain):
    """1-D DeviceMesh over the ranks of a reduction domain's process group."""
    from torch.distributed.device_mesh import DeviceMesh

    ranks = tuple(dist.get_process_group_ranks(domain.group) if domain.group is not None else range(dist.get_world_size()))
    key = (domain.device.type, ranks)
    if key not in _MESH_CACHE:
        _MESH_CACHE[key] = DeviceMesh(domain.device.type, list(ranks))
    return _MESH_CACHE[key]


def optimizer_state_for_dcp(engine, tp_rank: int = 0) -> dict:
    """Engine state with each bucket's shard as a DTensor (or a plain tensor for single-process runs)."""
    out = {"step": engine.step_count,
           "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in engine.param_groups]}
    for d in engine.domains:
        prefix = d.name if d.name != "tp_sharded" else f"tp_sharded.tp{tp_rank}"
        if d.name == "ep_experts":  # every expert-parallel rank owns different experts
            ep = getattr(engine.model, "_ep_ctx", None)
            prefix = f"ep_experts.ep{ep.rank if ep is not None else 0}"
        entry = {}
        for name, bufs in (("master", d.master), ("exp_avg", d.exp_avg), ("exp_avg_sq", d.exp_avg_sq)):
            for bi, t in enumerate(bufs):
                if dist.is_initialized() and d.size > 1:
                    from torch.distributed.tensor import DTensor, Replicate, Shard

                    placement = [Shard(0)] if d.shard else [Replicate()]
                    t = DTensor.from_local(t, _mesh_for(d), placement, run_check=False)
                entry[f"{name}.{bi}"] = t
        out[prefix] = entry
    return out


def load_optimizer_state_from_dcp(engine, state: dict, tp_rank: int = 0):
    engine.step_count = int(state["step"])
    for pg, saved in zip(engine.param_groups, state["param_groups"]):
        pg.update({k: v for k, v in saved.items() if k in ("lr", "initial_lr", "weight_decay")})
    # tensors were loaded in place (by DCP through the DTensors that wrap the engine's own buffers, or by the
    # resharding loader); the bf16 parameters follow the master copy
    engine.params_from_master()


# ----------------------------------------------------------------------------- save / load
def save_checkpoint(output_dir: str, step: int, model, engine, scheduler, counters: dict, tp_rank: int = 0) -> str:
    import torch.distributed.checkpoint as dcp

    path = checkpoint_dir(output_dir, step)
    state = {
        "model": model_state_for_save(model),
        "optimizer": optimizer_state_for_dcp(engine, tp_rank),
        "scheduler": {k: v for k, v in scheduler.state_dict().items() if k != "lr_lambdas"} if scheduler is not None else {},
        "step": int(step),
        "tokens_seen": int(counters.get("tokens_seen", 0)),
        "tokens_seen_assistant": int(counters.get("tokens_seen_assistant", 0)),
    }
    if not dist.is_initialized() or dist.get_rank() == 0:
        os.makedirs(path, exist_ok=True)
    if dist.is_initialized():
        dist.barrier()
    from . import opt_reshard

    tp = getattr(model, "tp", None)
    opt_reshard.write_layout(path, engine, tp.size if (tp is not None and tp.enabled) else 1)
    dcp.save(state, checkpoint_id=path, no_dist=not dist.is_initialized())
    logger.info(f"saved checkpoint {path}")
    return path


def load_checkpoint(output_dir: str, step: int, model, engine, scheduler, tp_rank: int = 0) -> dict:
    import torch.distributed.checkpoint as dcp

    path = checkpoint_dir(output_dir, step)
    if not os.path.exists(os.path.join(path, ".metadata")):
        raise FileNotFoundError(f"no complete checkpoint at {path}")
    if dist.is_initialized():
        dist.barrier()
    from . import opt_reshard

    shapes = _global_shapes(model)
    dev = next(model.parameters()).device
    model_buf = {k: torch.empty(shape, dtype=dt, device=dev) for k, (shape, dt) in shapes.items()}
    tp = getattr(model, "tp", None)
    saved_layout = opt_reshard.read_layout(path)
    here = opt_reshard.describe_layout(engine, tp.size if (tp is not None and tp.enabled) else 1)
    in_place = saved_layout is None or opt_reshard.same_layout(saved_layout, here)
    opt_state = optimizer_state_for_dcp(engine, tp_rank)
    if not in_place:
        # another parallel layout wrote this checkpoint: only the scalars load directly, the tensors are re-assembled
        opt_state = {"step": opt_state["step"], "param_groups": opt_state["param_groups"]}
    state = {
        "model": model_buf,
        "optimizer": opt_state,
        "scheduler": {k: v for k, v in scheduler.state_dict().items() if k != "lr_lambdas"} if scheduler is not None else {},
        "step": 0, "tokens_seen": 0, "tokens_seen_assistant": 0,
    }
    dcp.load(state, checkpoint_id=path, no_dist=not dist.is_initialized())
    load_model_state(model, state["model"])
    if not in_place:
        logger.info("the checkpoint was written under another parallel layout: re-assembling the optimizer state per parameter")
        opt_reshard.load_resharded(path, engine, saved_layout, tp)
    load_optimizer_state_from_dcp(engine, state["optimizer"], tp_rank)
    if scheduler is not None and state["scheduler"]:
        sd = scheduler.state_dict()
        sd.update({k: v for k, v in state["scheduler"].items() if k != "lr_lambdas"})
        scheduler.load_state_dict(sd)
    logger.info(f"loaded checkpoint {path} (step {state['step']})")
    return {"step": int(state["step"]), "tokens_seen": int(state["tokens_seen"]),
            "tokens_seen_assistant": int(state["tokens_seen_assistant"])}
