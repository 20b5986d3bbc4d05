"""Freeze policy and determinism (reference: train/utils.py:106-185)."""
from __future__ import annotations

import os

import torch


def set_model(model, train_llm: bool, train_mlp: bool, train_vit: bool):
    """``requires_grad`` by sub-tree: LLM (decoder + lm_head), MLP (merger + DeepStack mergers), ViT (the rest of
    ``visual``).  ``mtp.*`` parameters, where a model has them, stay frozen."""
    for name, p in model.named_parameters():
        if "visual.merger" in name or "visual.deepstack_merger_list" in name:
            p.requires_grad_(train_mlp)
        elif "visual." in name:
            p.requires_grad_(train_vit)
        elif name.startswith("mtp.") or ".mtp." in name:
            p.requires_grad_(False)
        else:
            p.requires_grad_(train_llm)
    return model


def set_determinism(seed: int, deterministic: bool = False):
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
