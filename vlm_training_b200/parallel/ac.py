"""Activation checkpointing for decoder / ViT blocks.

``full`` recomputes the whole block in backward; ``sac`` keeps the block's
mixer half (attention / Gated DeltaNet, whose recompute is the expensive part)
and recomputes only the MLP half, whose activations are the largest
(``DecoderLayer.forward_sac``; reference policy names: train/infra.py:155-234 —
there "sac" saves matmul outputs; here the custom ops decide what they save, so
the split is by sub-block).
"""
from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint


def checkpoint_layer(layer, x, ctx, mode: str):
    if mode == "full":
        return checkpoint(layer, x, ctx, use_reentrant=False)
    if mode == "sac":
        if not hasattr(layer, "forward_sac"):
            raise ValueError(f"ac_mode 'sac' needs a block with a forward_sac method; {type(layer).__name__} has none")
        return layer.forward_sac(x, ctx)
    return layer(x, ctx)


def apply_ac(model, mode: str, vision: bool = False):
    """Set the checkpoint policy on the model's decoder (and optionally its ViT;
    the reference never checkpoints the ViT, train/train_qwen.py:188-192)."""
    if mode not in ("off", "full", "sac"):
        raise ValueError(f"ac_mode must be off|full|sac, got {mode!r}")
    model.decoder.ac_mode = mode
    if vision and model.visual is not None:
        model.visual.ac_mode = mode
    return model
