"""Synthetic packed batches of the shapes the benchmark configurations name.

Every generator yields the batch dict the energon task encoders produce
(reference: data/energon_dataloader.py:321-337,431-464) — ``input_ids [L]``,
``attention_mask [L]``, ``cu_seqlens [n+1] int32``, ``labels [L]``,
``mm_token_type_ids [L]``, and for VLM rows ``pixel_values [N, C*Tp*P*P]`` and
``image_grid_thw [n_img, 3]`` — as CPU tensors, plus ``host`` with numpy copies
of the metadata the model needs (position ids, segment tables), computed here
so the training step itself never syncs with the device.

Labels follow the HF convention (``labels == input_ids``, the model shifts);
the first token of every document carries ``-100`` so the last token of one
document is not trained to predict the first token of the next.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from ..models import positions
from ..models.config import ModelConfig


@dataclass
class SyntheticSpec:
    kind: str = "text-loguniform"  # "text-uniform" | "text-loguniform" | "vlm"
    seq_len: int = 8192
    vocab_size: int = 151936
    doc_len_min: int = 128
    doc_len_max: int = 8192
    seed: int = 0
    # vlm
    images_min: int = 1
    images_max: int = 4
    side_min: int = 224
    side_max: int = 1024
    side_step: int = 32
    pixel_dtype: str = "bfloat16"


def _draw_len(rng: np.random.Generator, spec: SyntheticSpec) -> int:
    lo, hi = spec.doc_len_min, spec.doc_len_max
    if spec.kind == "text-uniform":
        return int(rng.integers(lo, hi + 1))
    return int(round(math.exp(rng.uniform(math.log(lo), math.log(hi)))))


def text_row(rng: np.random.Generator, spec: SyntheticSpec, vocab: int | None = None) -> dict:
    """One packed row of exactly ``seq_len`` tokens: documents are drawn until the row
    is full and the last one is cut to fit.  ``vocab``: ids are drawn below it (models with vision token ids pass the
    smallest special id so that text rows hold no image tokens)."""
    L = spec.seq_len
    cu = [0]
    while cu[-1] < L:
        cu.append(min(L, cu[-1] + max(1, _draw_len(rng, spec))))
    ids = rng.integers(0, vocab or spec.vocab_size, size=L, dtype=np.int64)
    labels = ids.copy()
    labels[np.asarray(cu[:-1])] = -100
    return {"input_ids": ids, "labels": labels, "cu_seqlens": np.asarray(cu, dtype=np.int32)}


def _text_vocab(spec: SyntheticSpec, cfg: ModelConfig) -> int:
    """Random text ids stay below every special (vision) token id and inside the vocabulary."""
    return max(1, min(spec.vocab_size, cfg.text.vocab_size, cfg.image_token_id, cfg.video_token_id,
                      cfg.vision_start_token_id, cfg.vision_end_token_id))


def _vlm_sample(rng, spec: SyntheticSpec, cfg: ModelConfig, budget: int):
    """Token ids / labels / grids of one multimodal sample that fits in ``budget`` tokens, or None."""
    merge = cfg.vision.spatial_merge_size
    patch = cfg.vision.patch_size
    n_img = int(rng.integers(spec.images_min, spec.images_max + 1))
    grids, img_tokens = [], []
    for _ in range(n_img):
        n_side = (spec.side_max - spec.side_min) // spec.side_step + 1
        h = (spec.side_min + spec.side_step * int(rng.integers(0, n_side))) // patch
        w = (spec.side_min + spec.side_step * int(rng.integers(0, n_side))) // patch
        grids.append((1, h, w))
        img_tokens.append((h // merge) * (w // merge))
    min_text = 4 * (n_img + 1)
    while grids and sum(img_tokens) + 2 * len(grids) + min_text > budget:
        grids.pop()
        img_tokens.pop()
    if not grids:
        return None
    fixed = sum(img_tokens) + 2 * len(grids)
    # text between images: uniform-random ids, lengths drawn so the sample stays inside the budget
    room = budget - fixed
    n_seg = len(grids) + 1
    want = min(room, int(rng.integers(4 * n_seg, max(4 * n_seg + 1, min(room, 64 * n_seg) + 1))))
    cuts = np.sort(rng.integers(0, want - 4 * n_seg + 1, size=n_seg - 1))
    seg = np.diff(np.concatenate(([0], cuts, [want - 4 * n_seg]))) + 4
    ids, labels = [], []
    for i in range(n_seg):
        t = rng.integers(0, _text_vocab(spec, cfg), size=int(seg[i]), dtype=np.int64)
        ids.append(t)
        labels.append(t.copy())
        if i < len(grids):
            blk = np.concatenate(([cfg.vision_start_token_id], np.full(img_tokens[i], cfg.image_token_id), [cfg.vision_end_token_id]))
            ids.append(blk.astype(np.int64))
            labels.append(np.full(blk.shape[0], -100, dtype=np.int64))
    ids, labels = np.concatenate(ids), np.concatenate(labels)
    labels[0] = -100
    return ids, labels, grids


def vlm_row(rng: np.random.Generator, spec: SyntheticSpec, cfg: ModelConfig) -> dict:
    """One packed multimodal row of exactly ``seq_len`` tokens.  Samples (1-4 images each, text in
    between) are appended while they fit; the tail is filled with one text-only document."""
    L = spec.seq_len
    ids_all, lab_all, grids_all, cu = [], [], [], [0]
    while cu[-1] < L:
        room = L - cu[-1]
        s = _vlm_sample(rng, spec, cfg, room) if room >= 64 + 2 + 16 else None
        if s is None:
            t = rng.integers(0, _text_vocab(spec, cfg), size=room, dtype=np.int64)
            lab = t.copy()
            lab[0] = -100
            ids_all.append(t)
            lab_all.append(lab)
            cu.append(L)
            break
        ids, labels, grids = s
        ids_all.append(ids)
        lab_all.append(labels)
        grids_all.extend(grids)
        cu.append(cu[-1] + ids.shape[0])
    ids = np.concatenate(ids_all)
    labels = np.concatenate(lab_all)
    grids = np.asarray(grids_all, dtype=np.int64).reshape(-1, 3)
    n_patches = int((grids[:, 0] * grids[:, 1] * grids[:, 2]).sum())
    # patches are drawn (with replacement) from a fixed pool of normal(0, 1) patch vectors: drawing 40 M fresh normals
    # per row costs about a second of host time, more than a training step, and would make the loader the bottleneck
    pool = _patch_pool(spec.seed, cfg.vision.patch_dim, spec.pixel_dtype)
    pixels = pool.index_select(0, torch.from_numpy(rng.integers(0, pool.shape[0], size=n_patches)))
    return {"input_ids": ids, "labels": labels, "cu_seqlens": np.asarray(cu, dtype=np.int32),
            "pixel_values": pixels, "image_grid_thw": grids}


_POOLS: dict = {}
_POOL_ROWS = 8192


def _patch_pool(seed: int, patch_dim: int, dtype: str) -> torch.Tensor:
    key = (seed, patch_dim, dtype)
    if key not in _POOLS:
        gen = torch.Generator().manual_seed(1000003 * seed + patch_dim)
        _POOLS[key] = torch.randn(_POOL_ROWS, patch_dim, generator=gen, dtype=torch.float32).to(getattr(torch, dtype))
    return _POOLS[key]


def host_plan(batch: dict, cfg: ModelConfig) -> dict:
    """numpy metadata for :class:`vlm_training_b200.models.BatchPlan` (built in the data workers)."""
    ids, cu = batch["input_ids"], batch["cu_seqlens"]
    T = ids.shape[0]
    grids = batch.get("image_grid_thw")
    out = {"max_seqlen": int(np.diff(cu).max())}
    if cfg.text.mrope_section is not None:
        out["position_ids"] = positions.mrope_position_ids(ids, cu, grids, cfg.image_token_id, cfg.video_token_id,
                                                           cfg.vision.spatial_merge_size if cfg.vision else 2)
    else:
        out["position_ids"] = positions.doc_position_ids(cu, T)[None]
    if cfg.text.is_hybrid:
        out["seq_idx"] = positions.seq_idx(cu, T)
    if grids is not None and len(grids):
        out["image_rows"] = np.flatnonzero(ids == cfg.image_token_id).astype(np.int64)
    return out


class SyntheticDataset:
    """Infinite iterator of packed rows; rank ``dp_rank`` of ``dp_size`` draws from its own stream
    (tensor-parallel peers pass the same ``dp_rank`` and so see identical data, as with the
    reference's energon ``WorkerConfig``, reference: train/train_qwen.py:227-232)."""

    def __init__(self, spec: SyntheticSpec, cfg: ModelConfig, dp_rank: int = 0, dp_size: int = 1, pad_token_id: int = 151643,
                 worker=(0, 1)):
        self.spec, self.cfg = spec, cfg
        # one random stream per (rank, worker); a single worker keeps the stream of the in-thread loader
        key = [spec.seed, dp_rank, dp_size] + ([int(worker[0]), int(worker[1])] if worker[1] > 1 else [])
        self.rng = np.random.default_rng(key)
        self.pad_token_id = pad_token_id

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        row = vlm_row(self.rng, self.spec, self.cfg) if self.spec.kind == "vlm" else text_row(self.rng, self.spec,
                                                                                                 _text_vocab(self.spec, self.cfg))
        host = host_plan(row, self.cfg)
        ids = torch.from_numpy(row["input_ids"])
        batch = {
            "input_ids": ids,
            "attention_mask": torch.ones_like(ids),
            "cu_seqlens": torch.from_numpy(row["cu_seqlens"]),
            "labels": torch.from_numpy(row["labels"]),
            "mm_token_type_ids": (ids == self.cfg.image_token_id).to(torch.int32),
            "host": host,
        }
        if "pixel_values" in row:
            batch["pixel_values"] = row["pixel_values"]
            batch["image_grid_thw"] = torch.from_numpy(row["image_grid_thw"])
        return batch


def spec_from_config(cfg_data, model_cfg: ModelConfig, seed: int = 0) -> SyntheticSpec:
    kind = cfg_data.synthetic
    if kind not in ("text-uniform", "text-loguniform", "vlm"):
        raise ValueError(f"data.synthetic must be text-uniform | text-loguniform | vlm, got {kind!r}")
    return SyntheticSpec(kind=kind, seq_len=int(cfg_data.seq_len), vocab_size=model_cfg.text.vocab_size,
                         doc_len_min=cfg_data.doc_len_min, doc_len_max=min(cfg_data.doc_len_max, int(cfg_data.seq_len)),
                         seed=seed)
