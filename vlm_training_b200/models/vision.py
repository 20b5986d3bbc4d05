"""Qwen3-VL / Qwen3.5 vision tower: patch embedding, ViT blocks with 2-D rotary
and per-frame bidirectional varlen attention, 2x2 spatial patch merger and
DeepStack mergers.  Module and parameter names follow the HF snapshot layout
(reference: models/qwen3_vl/model.py:336-600).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn

from .. import ops
from . import positions
from .config import VisionConfig
from .layers import Linear


@dataclass
class VisionPlan:
    """Host-built metadata for one batch of images (see :mod:`.positions`)."""

    cu_seqlens: torch.Tensor  # int32 [n_frames + 1]
    max_seqlen: int
    cos: torch.Tensor  # [N, head_dim] fp32
    sin: torch.Tensor
    pe_index: torch.Tensor  # int64 [4, N]
    pe_weight: torch.Tensor  # fp32 [4, N]

    @staticmethod
    def build(grids, cfg: VisionConfig, device) -> "VisionPlan":
        cu, mx = positions.vision_segments(grids)
        coords = positions.vision_rot_coords(grids, cfg.spatial_merge_size)
        half = cfg.head_dim // 2
        inv = 1.0 / (10000.0 ** (np.arange(0, half, 2, dtype=np.float32) / half))
        fr = coords[:, :, None].astype(np.float32) * inv[None, None, :]  # [N, 2, half/2]
        rot = fr.reshape(coords.shape[0], -1)  # [N, half]
        emb = np.concatenate((rot, rot), -1)
        side = int(round(cfg.num_position_embeddings ** 0.5))
        idx, wt = positions.vision_pos_embed_plan(grids, side, cfg.spatial_merge_size)
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=dt, non_blocking=True)
        return VisionPlan(t(cu, torch.int32), mx, t(np.cos(emb), torch.float32), t(np.sin(emb), torch.float32),
                          t(idx, torch.int64), t(wt, torch.float32))


class _PatchProj(nn.Module):
    """Conv3d with kernel == stride, i.e. a GEMM on flattened patches; the weight
    keeps the HF shape ``[hidden, C, Tp, P, P]``."""

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cfg.hidden_size, cfg.in_channels, cfg.temporal_patch_size,
                                               cfg.patch_size, cfg.patch_size))
        self.bias = nn.Parameter(torch.zeros(cfg.hidden_size))


class PatchEmbed(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.proj = _PatchProj(cfg)

    def forward(self, pixels):
        w = self.proj.weight
        return ops.linear(pixels.to(w.dtype), w.view(w.shape[0], -1), self.proj.bias)


class VisionAttention(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.n_heads, self.head_dim = cfg.num_heads, cfg.head_dim
        self.qkv = Linear(cfg.hidden_size, 3 * cfg.hidden_size, bias=True)
        self.proj = Linear(cfg.hidden_size, cfg.hidden_size, bias=True)

    def forward(self, x, plan: VisionPlan, prenorm: "nn.LayerNorm | None" = None):
        S = x.shape[0]
        if prenorm is not None:
            qkv = ops.layer_norm_linear(x, prenorm.weight, prenorm.bias, self.qkv.weight, self.qkv.bias, prenorm.eps)
        else:
            qkv = self.qkv(x)
        qkv = qkv.view(S, 3, self.n_heads, self.head_dim)
        q, k, v = qkv.unbind(1)
        D = self.head_dim
        # q and k leave the rotary kernel as contiguous [S, H, D]; v is read in place from the fused projection (the
        # attention kernels take strided heads and any head size that is a multiple of 8, 72 here)
        q, k = ops.rope_vision(q, k, plan.cos, plan.sin)
        o = ops.attention_varlen(q, k, v, plan.cu_seqlens, plan.max_seqlen, False, D ** -0.5)
        return self.proj(o.reshape(S, -1))


class VisionMLP(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.linear_fc1 = Linear(cfg.hidden_size, cfg.intermediate_size, bias=True)
        self.linear_fc2 = Linear(cfg.intermediate_size, cfg.hidden_size, bias=True)
        self.approx = "tanh" if "tanh" in cfg.hidden_act else "none"

    def forward(self, x, prenorm: "nn.LayerNorm | None" = None):
        if prenorm is not None:
            pre = ops.layer_norm_linear(x, prenorm.weight, prenorm.bias, self.linear_fc1.weight, self.linear_fc1.bias, prenorm.eps)
        else:
            pre = ops.linear(x, self.linear_fc1.weight, self.linear_fc1.bias)
        return ops.gelu_linear(pre, self.linear_fc2.weight, self.linear_fc2.bias, self.approx)


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.norm1 = nn.LayerNorm(cfg.hidden_size, eps=1e-6)
        self.norm2 = nn.LayerNorm(cfg.hidden_size, eps=1e-6)
        self.attn = VisionAttention(cfg)
        self.mlp = VisionMLP(cfg)

    def forward(self, x, plan: VisionPlan):
        x = x + self.attn(x, plan, prenorm=self.norm1)
        return x + self.mlp(x, prenorm=self.norm2)


class PatchMerger(nn.Module):
    """2x2 spatial merge MLP.  The main merger normalises each patch (dim
    ``hidden``) before grouping four of them; DeepStack mergers normalise the
    grouped vector (dim ``4*hidden``) (reference: models/qwen3_vl/model.py:446-462)."""

    def __init__(self, cfg: VisionConfig, postshuffle_norm: bool):
        super().__init__()
        self.merged = cfg.hidden_size * cfg.spatial_merge_size ** 2
        self.postshuffle = postshuffle_norm
        self.norm = nn.LayerNorm(self.merged if postshuffle_norm else cfg.hidden_size, eps=1e-6)
        self.linear_fc1 = Linear(self.merged, self.merged, bias=True)
        self.linear_fc2 = Linear(self.merged, cfg.out_hidden_size, bias=True)

    def forward(self, x):
        if self.postshuffle:
            x = ops.layer_norm(x.view(-1, self.merged), self.norm.weight, self.norm.bias, self.norm.eps)
        else:
            x = ops.layer_norm(x, self.norm.weight, self.norm.bias, self.norm.eps).view(-1, self.merged)
        pre = ops.linear(x, self.linear_fc1.weight, self.linear_fc1.bias)
        return ops.gelu_linear(pre, self.linear_fc2.weight, self.linear_fc2.bias, "none")


class VisionModel(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = PatchEmbed(cfg)
        self.pos_embed = nn.Embedding(cfg.num_position_embeddings, cfg.hidden_size)
        self.blocks = nn.ModuleList([VisionBlock(cfg) for _ in range(cfg.depth)])
        self.merger = PatchMerger(cfg, postshuffle_norm=False)
        self.deepstack_visual_indexes = list(cfg.deepstack_visual_indexes)
        self.deepstack_merger_list = nn.ModuleList(
            [PatchMerger(cfg, postshuffle_norm=True) for _ in self.deepstack_visual_indexes])
        self.ac_mode = "off"

    def forward(self, pixels, grid_thw=None, plan: VisionPlan | None = None):
        """pixels ``[N, C*Tp*P*P]`` in merge-block order → ``(merged [N/4, out], [deepstack...])``."""
        if plan is None:
            plan = VisionPlan.build(grid_thw.tolist() if torch.is_tensor(grid_thw) else grid_thw, self.cfg, pixels.device)
        x = self.patch_embed(pixels)
        pe = self.pos_embed.weight[plan.pe_index]  # [4, N, hidden]
        x = x + (pe.float() * plan.pe_weight.unsqueeze(-1)).sum(0).to(x.dtype)
        deep = []
        for i, blk in enumerate(self.blocks):
            if self.ac_mode != "off" and torch.is_grad_enabled():
                from ..parallel.ac import checkpoint_layer

                x = checkpoint_layer(blk, x, plan, "full")
            else:
                x = blk(x, plan)
            if i in self.deepstack_visual_indexes:
                deep.append(self.deepstack_merger_list[self.deepstack_visual_indexes.index(i)](x))
        return self.merger(x), deep
