"""Sequence packing primitives shared by the task encoders.

* ``assistant_label_mask``: train only on assistant turns — for every occurrence of the single
  token "assistant" at ``pos`` the span ``[pos+2, e+2)`` is kept, where ``e`` is the next EOS
  (so the EOS and the newline after it are trained) (reference: data/energon_dataloader.py:275-290).
* ``select_bins``: online packing of a buffer of encoded samples — sort by length (longest
  first), open a bin with the longest remaining sample, add every later sample that still
  fits, shuffle the bins (reference: data/energon_dataloader.py:410-428).  A sample longer than
  the row forms its own over-long bin.
* ``collate_row``: concatenate a bin into one row, ``cu_seqlens`` int32, right-pad to the row
  length and append the row length to ``cu_seqlens`` so the pad tail is its own attention
  segment (reference: data/energon_dataloader.py:431-464).
"""
from __future__ import annotations

import random

import numpy as np
import torch


def assistant_label_mask(input_ids, assistant_token: int, eos_token: int) -> torch.Tensor:
    ids = input_ids.tolist() if torch.is_tensor(input_ids) else list(input_ids)
    labels = torch.full((len(ids),), -100, dtype=torch.long)
    src = torch.as_tensor(ids, dtype=torch.long)
    pos, n = 0, len(ids)
    while pos < n:
        if ids[pos] == assistant_token:
            start = pos + 2
            end = start
            while end < n and ids[end] != eos_token:
                end += 1
            if end < n:
                labels[start:end + 2] = src[start:end + 2]
                pos = end
        pos += 1
    return labels


def select_bins(lengths: list[int], max_length: int, rng: random.Random | None = None) -> list[list[int]]:
    """Indices of the samples of each bin (first-fit over the length-sorted buffer)."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    used = [False] * len(order)
    bins = []
    for a, i in enumerate(order):
        if used[a]:
            continue
        used[a] = True
        cur, room = [i], max_length - lengths[i]
        for b in range(a + 1, len(order)):
            j = order[b]
            if not used[b] and lengths[j] <= room:
                used[b] = True
                cur.append(j)
                room -= lengths[j]
        bins.append(cur)
    (rng or random).shuffle(bins)
    return bins


def collate_row(samples: list[dict], max_length: int, pad_token_id: int) -> dict:
    """``samples``: dicts with ``input_ids``, ``labels`` and optionally ``attention_mask``,
    ``mm_token_type_ids``, ``pixel_values``, ``image_grid_thw`` (1-D / 2-D tensors)."""
    ids = torch.cat([s["input_ids"] for s in samples])
    labels = torch.cat([s["labels"] for s in samples])
    mask = torch.cat([s.get("attention_mask", torch.ones_like(s["input_ids"])) for s in samples])
    mm = torch.cat([s.get("mm_token_type_ids", torch.zeros_like(s["input_ids"], dtype=torch.int32)).to(torch.int32)
                    for s in samples])
    cu = [0] + np.cumsum([int(s["input_ids"].numel()) for s in samples]).tolist()
    pad = max_length - ids.numel()
    if pad > 0:
        ids = torch.cat((ids, torch.full((pad,), pad_token_id, dtype=ids.dtype)))
        labels = torch.cat((labels, torch.full((pad,), -100, dtype=labels.dtype)))
        mask = torch.cat((mask, torch.zeros(pad, dtype=mask.dtype)))
        mm = torch.cat((mm, torch.zeros(pad, dtype=mm.dtype)))
        cu.append(max_length)
    out = {"input_ids": ids, "attention_mask": mask, "cu_seqlens": torch.tensor(cu, dtype=torch.int32), "labels": labels,
           "mm_token_type_ids": mm}
    pix = [s["pixel_values"] for s in samples if s.get("pixel_values") is not None]
    if pix:
        out["pixel_values"] = torch.cat(pix, 0)
        out["image_grid_thw"] = torch.cat([s["image_grid_thw"].reshape(-1, 3) for s in samples if s.get("image_grid_thw") is not None], 0)
    return out
