"""Mark a model's linear layers for FP8 training.

The reference carries the same switch as ``apply_float8`` (reference: train/infra.py:139-153): torchao converts every
``nn.Linear`` whose name does not contain ``visual`` and whose dimensions are multiples of 16.  Here nothing is swapped:
the weight of every eligible :class:`~vlm_training_b200.models.layers.Linear` gets a tag, and ``ops.linear`` (and the fused
norm / activation + linear ops, which fall back to their unfused form for such a weight) sends a tagged weight through
``ops/float8.py``: tensor-wise dynamic scaling, e4m3 activations and weights, e5m2 output gradients, the three GEMMs on
the FP8 tensor cores.  Expert weights of the MoE layers (grouped GEMMs), the LM head (chunked linear + cross-entropy), the
DSA indexer's projections and the vision tower stay bf16.  With tensor parallelism the tagged layers use the plain
collectives around an FP8 GEMM instead of the bf16 GEMMs with the collective inside.
"""
from __future__ import annotations

import logging

import torch.nn as nn

log = logging.getLogger(__name__)


def eligible(name: str, module: nn.Module) -> bool:
    from ..models.layers import Linear

    leaf = name.split(".")[-1]
    if not isinstance(module, Linear) or "visual" in name or leaf == "lm_head" or leaf.startswith("idx_"):
        return False   # idx_*: the DSA indexer ranks keys for a top-k selection and keeps its precision
    w = module.weight
    return w.dim() == 2 and w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0


def apply_float8(model: nn.Module) -> list[str]:
    """Tag the eligible linears of ``model``; returns their names."""
    names = []
    for name, module in model.named_modules():
        if eligible(name, module):
            module.weight._vlmt_fp8 = True
            names.append(name)
    log.info("float8: %d linear layers run their GEMMs in FP8", len(names))
    return names


def remove_float8(model: nn.Module) -> None:
    for p in model.parameters():
        if getattr(p, "_vlmt_fp8", False):
            p._vlmt_fp8 = False
