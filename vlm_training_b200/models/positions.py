"""Host-side builders for everything the models derive from ``cu_seqlens``,
``input_ids`` and ``image_grid_thw``.

The reference computes these inside ``forward`` with Python loops over device
tensors (``.tolist()`` / ``.item()`` syncs every step; reference:
models/qwen3_vl/model.py:488-571,644-713,765).  Here they are plain numpy
functions run by the data pipeline (or once per batch by the model when the
caller did not supply them), so the training step never waits on the GPU.
"""
from __future__ import annotations

import numpy as np


# ----------------------------------------------------------------------------- text
def doc_position_ids(cu_seqlens, total: int) -> np.ndarray:
    """Per-document ``arange`` positions for a packed row, ``[total]`` int64.
    Tokens past the last boundary continue the count from zero."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    pos = np.arange(total, dtype=np.int64)
    starts = np.zeros(total, dtype=np.int64)
    inner = cu[1:-1]
    inner = inner[(inner > 0) & (inner < total)]
    if len(inner):
        seg = np.searchsorted(inner, pos, side="right")
        bounds = np.concatenate(([0], inner))
        starts = bounds[seg]
    return pos - starts


def seq_idx(cu_seqlens, total: int) -> np.ndarray:
    """Document index of every token (``#{inner boundaries <= t}``), int32."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    return np.searchsorted(cu[1:-1], np.arange(total), side="right").astype(np.int32)


def mrope_position_ids(input_ids, cu_seqlens, grids, image_token_id: int, video_token_id: int,
                       merge: int = 2, video_grids=None) -> np.ndarray:
    """3-axis (t, h, w) rotary positions of one packed row → ``[3, T]`` int64.

    Walk each document ``[cu[i], cu[i+1])`` with ``current = 0``.  A run of text
    tokens of length L gets ``current + arange(L)`` on all axes and advances
    ``current`` by L.  A run of image (video) placeholder tokens consumes the
    next image (video-frame) grid ``(t, h, w)``: temporal axis = ``current``,
    height axis = ``current + row``, width axis = ``current + col`` over the
    ``(h/merge, w/merge)`` merged grid, and ``current`` advances by
    ``max(h/merge, w/merge)``.  Video grids are expanded to ``t`` single-frame
    grids first.  One run is one grid: images are separated by text tokens
    (reference: models/qwen3_vl/model.py:644-713)."""
    ids = np.asarray(input_ids).reshape(-1)
    T = ids.shape[0]
    cu = [int(c) for c in np.asarray(cu_seqlens).reshape(-1)]
    if cu[-1] < T:
        cu = cu + [T]
    out = np.zeros((3, T), dtype=np.int64)
    kind = np.zeros(T, dtype=np.int8)
    kind[ids == image_token_id] = 1
    kind[ids == video_token_id] = 2
    if not kind.any():
        out[:] = doc_position_ids(cu, T)
        return out
    img = [tuple(int(v) for v in g) for g in np.asarray(grids if grids is not None else []).reshape(-1, 3).tolist()]
    vid = []
    for t, h, w in np.asarray(video_grids if video_grids is not None else []).reshape(-1, 3).tolist():
        vid.extend([(1, int(h), int(w))] * int(t))
    nxt = {1: 0, 2: 0}
    pools = {1: img, 2: vid}
    change = np.flatnonzero(np.diff(kind)) + 1
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        lo, hi = np.searchsorted(change, s, side="right"), np.searchsorted(change, e, side="left")
        cuts = [s] + [int(c) for c in change[lo:hi]] + [e]
        current = 0
        for a, b in zip(cuts[:-1], cuts[1:]):
            L, kd = b - a, int(kind[a])
            if kd == 0:
                out[:, a:b] = current + np.arange(L)
                current += L
                continue
            t, h, w = pools[kd][nxt[kd]]
            nxt[kd] += 1
            lh, lw = h // merge, w // merge
            if L != t * lh * lw:
                raise ValueError(f"vision run of {L} tokens at {a} does not match grid {(t, h, w)} -> {t * lh * lw}")
            out[0, a:b] = current
            out[1, a:b] = current + np.tile(np.repeat(np.arange(lh), lw), t)
            out[2, a:b] = current + np.tile(np.tile(np.arange(lw), lh), t)
            current += max(lh, lw)
    return out


# ----------------------------------------------------------------------------- vision
def vision_segments(grids) -> tuple[np.ndarray, int]:
    """ViT attention segments: one per (image, frame) of ``h*w`` patches
    (reference: models/qwen3_vl/model.py:585-590).  Returns (cu int32, max_seqlen)."""
    g = np.asarray(grids, dtype=np.int64).reshape(-1, 3)
    lens = np.repeat(g[:, 1] * g[:, 2], g[:, 0])
    cu = np.concatenate(([0], np.cumsum(lens))).astype(np.int32)
    return cu, int(lens.max()) if len(lens) else 0


def vision_rot_coords(grids, merge: int = 2) -> np.ndarray:
    """(row, col) of every patch in merge-block order, ``[N, 2]`` int64
    (reference: models/qwen3_vl/model.py:488-516)."""
    out = []
    for t, h, w in np.asarray(grids, dtype=np.int64).reshape(-1, 3).tolist():
        mh, mw = h // merge, w // merge
        r = (np.arange(mh)[:, None, None, None] * merge + np.arange(merge)[None, None, :, None])
        c = (np.arange(mw)[None, :, None, None] * merge + np.arange(merge)[None, None, None, :])
        r = np.broadcast_to(r, (mh, mw, merge, merge)).reshape(-1)
        c = np.broadcast_to(c, (mh, mw, merge, merge)).reshape(-1)
        rc = np.stack((r, c), -1)
        out.append(np.tile(rc, (t, 1)) if t > 1 else rc)
    return np.concatenate(out, 0) if out else np.zeros((0, 2), dtype=np.int64)


def vision_pos_embed_plan(grids, num_grid_per_side: int, merge: int = 2) -> tuple[np.ndarray, np.ndarray]:
    """Bilinear resampling of the learned ``side x side`` position table onto each
    image's ``h x w`` patch grid, emitted in merge-block order.

    Returns ``(index [4, N] int64, weight [4, N] float32)``: patch n gets
    ``sum_c weight[c, n] * table[index[c, n]]``
    (reference: models/qwen3_vl/model.py:518-571)."""
    idx_out, w_out = [], []
    side = num_grid_per_side
    for t, h, w in np.asarray(grids, dtype=np.int64).reshape(-1, 3).tolist():
        hi = np.linspace(0, side - 1, h, dtype=np.float32)
        wi = np.linspace(0, side - 1, w, dtype=np.float32)
        hf, wf = hi.astype(np.int64), wi.astype(np.int64)
        hc, wc = np.minimum(hf + 1, side - 1), np.minimum(wf + 1, side - 1)
        dh, dw = hi - hf, wi - wf
        idx = np.stack([
            (hf[:, None] * side + wf[None]).reshape(-1), (hf[:, None] * side + wc[None]).reshape(-1),
            (hc[:, None] * side + wf[None]).reshape(-1), (hc[:, None] * side + wc[None]).reshape(-1)], 0)
        wt = np.stack([
            ((1 - dh)[:, None] * (1 - dw)[None]).reshape(-1), ((1 - dh)[:, None] * dw[None]).reshape(-1),
            (dh[:, None] * (1 - dw)[None]).reshape(-1), (dh[:, None] * dw[None]).reshape(-1)], 0).astype(np.float32)

        def reorder(a):
            a = np.tile(a.reshape(4, 1, h, w), (1, t, 1, 1))
            a = a.reshape(4, t, h // merge, merge, w // merge, merge).transpose(0, 1, 2, 4, 3, 5)
            return a.reshape(4, -1)

        idx_out.append(reorder(idx))
        w_out.append(reorder(wt))
    if not idx_out:
        return np.zeros((4, 0), dtype=np.int64), np.zeros((4, 0), dtype=np.float32)
    return np.concatenate(idx_out, 1), np.concatenate(w_out, 1)


def num_image_tokens(grids, merge: int = 2) -> int:
    g = np.asarray(grids, dtype=np.int64).reshape(-1, 3)
    return int((g[:, 0] * (g[:, 1] // merge) * (g[:, 2] // merge)).sum())


def assign_images(grids, parts: int) -> list[list[int]]:
    """Image indices per part, balanced by the vision tower's cost per image (linear layers ~ patches, attention ~
    patches^2): longest-processing-time-first assignment.  Within a part the images keep their original order.
    Contiguous ranges balanced by patch count alone leave the parts about 5 % apart on rows of ~19 images
    (up to one 4096-patch image); this assignment brings that under 1 %."""
    g = np.asarray(grids, dtype=np.int64).reshape(-1, 3)
    n = g[:, 0] * g[:, 1] * g[:, 2]
    cost = n.astype(np.float64) + n.astype(np.float64) ** 2 / 6000.0
    load = np.zeros(parts)
    out: list[list[int]] = [[] for _ in range(parts)]
    for i in np.argsort(-cost, kind="stable"):
        p = int(np.argmin(load))
        load[p] += cost[i]
        out[p].append(int(i))
    return [sorted(ix) for ix in out]
