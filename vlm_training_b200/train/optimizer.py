"""Optimizer parameter groups and construction.

Three learning-rate groups by parameter name: merger + DeepStack mergers → ``lr_mlp``;
``visual.patch_embed`` / ``visual.pos_embed`` / ``visual.blocks`` → ``lr_vit``; everything
else → ``lr_llm``.  This is what the reference intends; its code puts every non-merger
parameter into the ``lr_mlp`` group because of a truthy-string condition
(reference: train/train_qwen.py:281-312), which is not reproduced.  One-dimensional
parameters (norm weights, biases, A_log, dt_bias) get no weight decay.
"""
from __future__ import annotations

import torch

from ..parallel.engine import GroupSpec, ShardedOptimizerEngine


def group_of(name: str) -> str:
    if "visual.merger" in name or "visual.deepstack_merger_list" in name:
        return "mlp"
    if "visual." in name:
        return "vit"
    return "llm"


def build_param_groups(model, lr_llm: float, lr_mlp: float, lr_vit: float, weight_decay: float) -> list[GroupSpec]:
    buckets: dict[tuple[str, bool], list] = {}
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        decay = p.dim() >= 2
        buckets.setdefault((group_of(name), decay), []).append(p)
    lrs = {"llm": lr_llm, "mlp": lr_mlp, "vit": lr_vit}
    groups = []
    for kind in ("llm", "mlp", "vit"):
        for decay in (True, False):
            ps = buckets.get((kind, decay))
            if ps:
                groups.append(GroupSpec(name=f"{kind}{'' if decay else '_nodecay'}", params=ps, lr=lrs[kind],
                                        weight_decay=weight_decay if decay else 0.0))
    return groups


def create_optimizer(model, tcfg, mesh, *, fused_comm: bool = False) -> ShardedOptimizerEngine:
    groups = build_param_groups(model, tcfg.lr_llm, tcfg.lr_mlp, tcfg.lr_vit, tcfg.weight_decay)
    return ShardedOptimizerEngine(
        model, groups, dp_group=mesh.dp_group, world_group=mesh.world_group, tp_size=mesh.tp,
        mode="fsdp" if tcfg.data_parallel == "fsdp" else "ddp", betas=(tcfg.beta1, tcfg.beta2), eps=tcfg.eps,
        max_grad_norm=tcfg.max_grad_norm if tcfg.clip_grad else None,
        state_dtype=torch.bfloat16 if tcfg.optimizer_state_dtype == "bf16" else torch.float32,
        fused_comm=fused_comm, reshard=bool(getattr(tcfg, "reshard_params", False)),
        reshard_after_forward=bool(getattr(tcfg, "reshard_after_forward", True)),
        fuse_first_gemm=bool(getattr(tcfg, "reshard_fuse_first_gemm", True)))
