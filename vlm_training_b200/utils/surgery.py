"""Weight surgery at start-up: graft a text-only checkpoint into the VLM's decoder and a SigLIP2 vision
encoder into the Qwen3-VL ViT (reference: train/utils.py:295-485)."""
from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F

from ..models.loader import snapshot_files


def _iter_snapshot(model_dir: str):
    from safetensors import safe_open

    for path in snapshot_files(model_dir):
        with safe_open(path, framework="pt", device="cpu") as fh:
            for key in fh.keys():
                yield key, fh.get_tensor(key)


def load_text_model(model, text_model_dir: str) -> int:
    """Copy a text-only snapshot (``model.*`` / ``lm_head.weight``) into ``model.language_model.*``.  When the
    vocabularies differ, the shared leading rows of ``embed_tokens`` / ``lm_head`` are copied
    (reference: train/utils.py:424-485)."""
    target = model.state_dict()
    n = 0
    with torch.no_grad():
        for key, src in _iter_snapshot(text_model_dir):
            name = key
            if key.startswith("model.") and not key.startswith("model.language_model."):
                name = "model.language_model." + key[len("model."):]
            if name not in target:
                continue
            dst = target[name]
            if dst.shape != src.shape:
                if dst.dim() == 2 and dst.shape[1] == src.shape[1] and ("embed_tokens" in name or "lm_head" in name):
                    rows = min(dst.shape[0], src.shape[0])
                    dst[:rows].copy_(src[:rows].to(dst.dtype))
                    n += 1
                    continue
                raise ValueError(f"shape mismatch for {name}: {tuple(src.shape)} vs {tuple(dst.shape)}")
            dst.copy_(src.to(dst.dtype))
            n += 1
    if n == 0:
        raise RuntimeError(f"no tensor of {text_model_dir} matched the decoder")
    return n


def load_vision_model(model, vision_model_dir: str) -> int:
    """SigLIP2 → Qwen3-VL ViT (reference: train/utils.py:295-422): the Conv2d patch embedding is inflated to the
    temporal Conv3d (weight repeated over the temporal patch and divided by its size), the learned position table
    is bilinearly resized to the ViT's grid, separate q/k/v projections are fused, names are mapped, and the
    merger / DeepStack mergers are Xavier-initialised."""
    vis = model.visual
    if vis is None:
        raise ValueError("the model has no vision tower")
    cfg = vis.cfg
    sd = {}
    for key, t in _iter_snapshot(vision_model_dir):
        k = key
        for pre in ("vision_model.", "model.vision_model."):
            if k.startswith(pre):
                k = k[len(pre):]
        sd[k] = t
    tgt = vis.state_dict()
    n = 0
    with torch.no_grad():
        w = sd.get("embeddings.patch_embedding.weight")
        if w is not None:
            if w.dim() == 2:  # NaFlex stores a linear patch embedding [hidden, C*P*P]
                w = w.view(w.shape[0], cfg.in_channels, cfg.patch_size, cfg.patch_size)
            w3 = w.unsqueeze(2).repeat(1, 1, cfg.temporal_patch_size, 1, 1) / cfg.temporal_patch_size
            tgt["patch_embed.proj.weight"].copy_(w3.to(tgt["patch_embed.proj.weight"].dtype))
            tgt["patch_embed.proj.bias"].copy_(sd["embeddings.patch_embedding.bias"])
            n += 2
        pe = sd.get("embeddings.position_embedding.weight")
        if pe is not None:
            side_src = int(round(math.sqrt(pe.shape[0])))
            side_dst = int(round(math.sqrt(cfg.num_position_embeddings)))
            grid = pe.float().view(1, side_src, side_src, -1).permute(0, 3, 1, 2)
            grid = F.interpolate(grid, size=(side_dst, side_dst), mode="bilinear", align_corners=False)
            tgt["pos_embed.weight"].copy_(grid.permute(0, 2, 3, 1).reshape(side_dst * side_dst, -1))
            n += 1
        for j in range(cfg.depth):
            src = f"encoder.layers.{j}."
            if src + "self_attn.q_proj.weight" not in sd:
                continue
            for suffix in ("weight", "bias"):
                qkv = torch.cat([sd[f"{src}self_attn.{p}_proj.{suffix}"] for p in ("q", "k", "v")], 0)
                tgt[f"blocks.{j}.attn.qkv.{suffix}"].copy_(qkv)
                tgt[f"blocks.{j}.attn.proj.{suffix}"].copy_(sd[f"{src}self_attn.out_proj.{suffix}"])
                tgt[f"blocks.{j}.norm1.{suffix}"].copy_(sd[f"{src}layer_norm1.{suffix}"])
                tgt[f"blocks.{j}.norm2.{suffix}"].copy_(sd[f"{src}layer_norm2.{suffix}"])
                tgt[f"blocks.{j}.mlp.linear_fc1.{suffix}"].copy_(sd[f"{src}mlp.fc1.{suffix}"])
                tgt[f"blocks.{j}.mlp.linear_fc2.{suffix}"].copy_(sd[f"{src}mlp.fc2.{suffix}"])
                n += 6
    from ..models.init import init_qwen3vl_

    init_qwen3vl_(model, seed=42)
    if n == 0:
        raise RuntimeError(f"no tensor of {vision_model_dir} matched the vision tower")
    return n
