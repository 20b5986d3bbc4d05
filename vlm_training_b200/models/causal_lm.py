"""Top-level models: Qwen3 (text), Qwen3-VL and Qwen3.5 (hybrid, dense or MoE).

All three share the forward contract of the reference VLM models
(reference: models/qwen3_vl/model.py:721-841, models/qwen3_5/model.py:674-760):

* ``input_ids``  one packed row, ``[T]`` or ``[1, T]``;
* ``attention_mask`` IS ``cu_seqlens`` (1-D, starts at 0, ends at T); ``None`` =
  one document;
* ``labels`` ``[T]``/``[1, T]`` → returns ``CausalLMOutput(loss, logits)``; the
  loss is the mean next-token cross-entropy over labels != -100, computed by
  the chunked linear+CE op so the ``[T, V]`` logits are never materialised
  (``logits`` is None unless ``return_logits=True``);
* ``pixel_values`` ``[N_patches, C*Tp*P*P]`` in merge-block order and
  ``image_grid_thw [n_img, 3]``.

State-dict keys follow the HF snapshots: ``model.*`` / ``lm_head.weight`` for
text Qwen3, ``model.language_model.*`` / ``model.visual.*`` / ``lm_head.weight``
for the VLMs.  ``batch_plan`` (a :class:`BatchPlan`) carries host-precomputed
metadata so ``forward`` performs no device→host sync; without it the model
builds one itself (one sync per batch).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch
import torch.nn as nn

from .. import ops
from . import positions
from .config import ModelConfig, TextConfig
from .layers import Decoder, Linear, RowContext
from .vision import VisionModel, VisionPlan


@dataclass
class CausalLMOutput:
    loss: torch.Tensor | None
    logits: torch.Tensor | None
    loss_sum: torch.Tensor | None = None
    n_valid: torch.Tensor | None = None


@dataclass
class BatchPlan:
    """Everything ``forward`` needs besides the tensors themselves, built on the
    host from numpy copies of the batch."""

    cu_seqlens: torch.Tensor  # int32 device
    max_seqlen: int
    position_ids: torch.Tensor  # int64 [3, T] (or [1, T] for text) device
    seq_idx: torch.Tensor | None = None  # int32 [T]
    image_rows: torch.Tensor | None = None  # int64 rows of the packed sequence that hold image tokens
    vision: VisionPlan | None = None
    extras: dict = field(default_factory=dict)
    image_rows_host: np.ndarray | None = None

    def local_image_rows(self, lo: int, hi: int, device):
        """(indices into the vision features, row indices local to the token shard [lo, hi))."""
        rows = self.image_rows_host
        sel = np.flatnonzero((rows >= lo) & (rows < hi))
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=torch.int64, non_blocking=True)
        return t(sel), t(rows[sel] - lo)

    @staticmethod
    def build(cfg: ModelConfig, input_ids, cu_seqlens, grids, device, need_seq_idx: bool | None = None) -> "BatchPlan":
        ids = np.asarray(input_ids.cpu() if torch.is_tensor(input_ids) else input_ids).reshape(-1)
        T = ids.shape[0]
        cu = np.asarray(cu_seqlens.cpu() if torch.is_tensor(cu_seqlens) else cu_seqlens, dtype=np.int64).reshape(-1) \
            if cu_seqlens is not None else np.array([0, T], dtype=np.int64)
        lens = np.diff(cu)
        mx = int(lens.max()) if len(lens) else T
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=dt, non_blocking=True)
        grids_l = None
        if grids is not None:
            grids_l = (grids.cpu().tolist() if torch.is_tensor(grids) else np.asarray(grids).tolist())
        if cfg.text.mrope_section is not None:
            pos = positions.mrope_position_ids(ids, cu, grids_l, cfg.image_token_id, cfg.video_token_id,
                                               cfg.vision.spatial_merge_size if cfg.vision else 2)
        else:
            pos = positions.doc_position_ids(cu, T)[None]
        plan = BatchPlan(t(cu, torch.int32), mx, t(pos, torch.int64))
        plan.extras["cu_host"] = cu.tolist()
        if need_seq_idx if need_seq_idx is not None else cfg.text.is_hybrid:
            plan.seq_idx = t(positions.seq_idx(cu, T), torch.int32)
        if grids_l:
            rows = np.flatnonzero(ids == cfg.image_token_id)
            plan.image_rows = t(rows, torch.int64)
            plan.image_rows_host = rows
            plan.vision = VisionPlan.build(grids_l, cfg.vision, device)
        return plan


def rotary_inv_freq(cfg: TextConfig, device=None) -> torch.Tensor:
    r = cfg.rope_dim
    return 1.0 / (cfg.rope_theta ** (torch.arange(0, r, 2, dtype=torch.float32, device=device) / r))


def rotary_tables(cfg: TextConfig, position_ids, inv_freq, dtype):
    """cos/sin ``[T, R]`` from ``position_ids`` (``[3, T]`` MRoPE or ``[1, T]`` text)."""
    if cfg.mrope_section is not None:
        if position_ids.shape[0] == 1:
            position_ids = position_ids.expand(3, -1)
        return ops.ref.mrope_cos_sin(position_ids, inv_freq, cfg.mrope_section, dtype)
    f = position_ids[0].float().unsqueeze(-1) * inv_freq.float()
    emb = torch.cat((f, f), -1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


class _CausalLMBase(nn.Module):
    config: ModelConfig
    ce_chunk_size: int = 1024

    # -- sub-module access (same for every family) --------------------------
    @property
    def decoder(self) -> Decoder:
        raise NotImplementedError

    @property
    def visual(self) -> VisionModel | None:
        return None

    def output_weight(self):
        return self.decoder.embed_tokens.weight if self.config.text.tie_word_embeddings else self.lm_head.weight

    # -- shared forward ------------------------------------------------------
    def forward(self, input_ids, attention_mask=None, labels=None, pixel_values=None, image_grid_thw=None,
                batch_plan: BatchPlan | None = None, return_logits: bool | None = None, **_ignored):
        cfg = self.config
        ids = input_ids.reshape(-1)
        T = ids.shape[0]
        if input_ids.dim() == 2 and input_ids.shape[0] != 1:
            raise ValueError("one packed row per call: the batch dimension must be 1")
        dec = self.decoder
        dev = dec.embed_tokens.weight.device
        if cfg.vision is not None and max(cfg.image_token_id, cfg.vision_start_token_id, cfg.vision_end_token_id) >= cfg.text.vocab_size:
            raise ValueError("the vision token ids lie outside the vocabulary; an embedding lookup with them would be out of range")
        if batch_plan is None:
            batch_plan = BatchPlan.build(cfg, ids, attention_mask, image_grid_thw if pixel_values is not None else None, dev)
        if ids.is_cuda:
            from ..ops import cuda as _cu

            if _cu.debug_checks_enabled():
                _cu.validate_row_indices(batch_plan.cu_seqlens, T, batch_plan.image_rows)
        tp = getattr(self, "tp", None)
        sp = tp is not None and tp.enabled and tp.sequence_parallel
        if tp is not None and tp.p2p is not None and torch.is_grad_enabled():
            # peers store this pass's gathered activations into buffers that the previous backward pass still read
            tp.p2p.begin_microbatch()
        lo, hi = 0, T
        if sp:
            if T % tp.size:
                raise ValueError(f"sequence parallelism needs the row length ({T}) divisible by tp={tp.size}")
            lo, hi = tp.rank * (T // tp.size), (tp.rank + 1) * (T // tp.size)
        x = ops.embedding(ids[lo:hi], dec.embed_tokens.weight)
        deepstack = None
        if pixel_values is not None and self.visual is not None:
            if tp is not None and tp.enabled:
                merged, deep = self._vision_image_parallel(pixel_values, image_grid_thw, tp, dev)
            else:
                merged, deep = self.visual(pixel_values, image_grid_thw, batch_plan.vision)
            rows = batch_plan.image_rows
            if rows.numel() != merged.shape[0]:
                raise ValueError(f"{rows.numel()} image tokens in the row but the vision tower produced {merged.shape[0]}")
            if sp:
                # keep the image tokens that fall in this rank's token shard (selection built on the host)
                sel, local_rows = batch_plan.local_image_rows(lo, hi, dev)
                merged, deep, rows = merged[sel], [d[sel] for d in deep], local_rows
            x = ops.scatter_rows(x, rows, merged)
            deepstack = [(rows, d) for d in deep]
        inv_freq = self._inv_freq(dev)
        cos, sin = rotary_tables(cfg.text, batch_plan.position_ids, inv_freq, torch.float32)
        ctx = RowContext(batch_plan.cu_seqlens, batch_plan.max_seqlen, cos, sin, batch_plan.seq_idx, batch_plan.extras)
        x = self._run_decoder(x, ctx, deepstack, batch_plan)
        want_logits = return_logits if return_logits is not None else labels is None
        logits = None
        if want_logits:
            logits = ops.linear(x, self.output_weight())
            if sp:
                from ..parallel.tp_comm import gather_rows

                logits = gather_rows(logits, tp)
            logits = logits.unsqueeze(0)
        if labels is None:
            return logits
        lab = labels.reshape(-1)
        targets = torch.cat((lab[1:], lab.new_full((1,), -100)))  # next-token shift over the whole row
        loss_sum, n_valid = self._loss(x, targets[lo:hi])
        if sp:
            from ..parallel.tp_comm import _ReduceFromTP

            loss_sum = _ReduceFromTP.apply(loss_sum.reshape(1), tp).reshape(())
            n_valid = (targets != -100).sum()
        loss = loss_sum / n_valid.to(loss_sum.dtype)
        return CausalLMOutput(loss=loss, logits=logits, loss_sum=loss_sum, n_valid=n_valid)

    def _vision_image_parallel(self, pixel_values, image_grid_thw, tp, dev):
        """The vision tower is replicated across the tensor-parallel group (as in the reference,
        train/infra.py:382-383) but its WORK is not: every rank encodes a contiguous share of the row's images
        and the merged / DeepStack features are exchanged with one uneven all-gather (the backward of which
        routes each feature's gradient back to the rank that produced it)."""
        from ..parallel.tp_comm import gather_uneven

        grids = image_grid_thw.tolist() if torch.is_tensor(image_grid_thw) else list(image_grid_thw)
        merge2 = self.config.vision.spatial_merge_size ** 2
        assign = positions.assign_images(grids, tp.size)          # image indices per rank, balanced by cost
        n_patch = [t * h * w for t, h, w in grids]
        p_off = [0]
        for n in n_patch:
            p_off.append(p_off[-1] + n)
        mine = assign[tp.rank]
        if mine:
            plan = VisionPlan.build([grids[i] for i in mine], self.config.vision, dev)
            pix = torch.cat([pixel_values[p_off[i]:p_off[i + 1]] for i in mine], 0) if len(mine) > 1 else \
                pixel_values[p_off[mine[0]]:p_off[mine[0] + 1]]
            merged, deep = self.visual(pix, None, plan)
            feats = torch.cat([merged] + list(deep), dim=-1)
        else:
            # A rank without images still runs the tower, on one dummy image of 2 x 2 patches whose features are dropped:
            # every rank then executes the same modules in the same order, so the collectives that belong to the tower's
            # parameters (bucket reductions from the gradient hooks, parameter gathers of sharded units) line up across
            # ranks, and the exchange's backward collective stays in this rank's autograd graph.
            ms = self.config.vision.spatial_merge_size
            dummy = [[1, ms, ms]]
            plan = VisionPlan.build(dummy, self.config.vision, dev)
            pix = pixel_values.new_zeros((ms * ms, pixel_values.shape[1]))
            merged, deep = self.visual(pix, None, plan)
            feats = torch.cat([merged] + list(deep), dim=-1)[:0]
        sizes = [sum(n_patch[i] for i in ix) // merge2 for ix in assign]
        allf = gather_uneven(feats, sizes, tp, grad_identical=not tp.sequence_parallel)
        # the gathered rows are rank-major; put the images back in their order of appearance in the row
        tok_of = [n // merge2 for n in n_patch]
        start_in_gather, pos = {}, 0
        for ix in assign:
            for i in ix:
                start_in_gather[i] = pos
                pos += tok_of[i]
        if [i for ix in assign for i in ix] != list(range(len(grids))):
            order = np.concatenate([np.arange(start_in_gather[i], start_in_gather[i] + tok_of[i]) for i in range(len(grids))])
            allf = allf.index_select(0, torch.from_numpy(order).to(dev, non_blocking=True))
        H = self.config.vision.out_hidden_size
        chunks = allf.split(H, dim=-1)
        return chunks[0], list(chunks[1:])

    def _run_decoder(self, x, ctx, deepstack, batch_plan):
        return self.decoder.run_layers(x, ctx, deepstack)

    def _loss(self, hidden, targets):
        return ops.linear_cross_entropy(hidden, self.output_weight(), targets, self.ce_chunk_size)

    def _inv_freq(self, device):
        buf = getattr(self, "_inv_freq_cache", None)
        if buf is None or buf.device != torch.device(device):
            buf = rotary_inv_freq(self.config.text, device)
            self._inv_freq_cache = buf
        return buf

    # -- construction helpers -------------------------------------------------
    @classmethod
    def from_config(cls, config: ModelConfig, dtype=torch.float32, device="cpu", init: bool = True, seed: int = 0):
        with torch.device("meta"):
            model = cls(config)
        model = model.to_empty(device=device).to(dtype)
        if init:
            from .init import init_normal_

            init_normal_(model, std=0.02, seed=seed)
        return model

    @classmethod
    def from_pretrained(cls, model_dir, dtype=torch.bfloat16, device="cpu", load_vision: bool = True):
        """Meta-init, materialise on ``device`` and stream a safetensors snapshot in
        (reference: models/qwen3_vl/model.py:843-949).  Returns ``(model, config)``."""
        import os

        from .loader import load_snapshot_into

        config = ModelConfig.from_json(os.path.join(model_dir, "config.json"))
        with torch.device("meta"):
            model = cls(config)
        model = model.to_empty(device=device).to(dtype)
        from .init import init_normal_

        init_normal_(model, std=0.02, seed=0, only_uninitialised=False)
        skip = ("model.visual.",) if not load_vision else ()
        load_snapshot_into(model, model_dir, dtype=dtype, allow_missing_prefixes=skip,
                           tied=config.text.tie_word_embeddings)
        return model, config


class _TextBackbone(nn.Module):
    """Gives the text model the HF prefix ``model.`` (``model.embed_tokens`` ...)."""


class Qwen3ForCausalLM(_CausalLMBase):
    """Text-only Qwen3 with varlen packing and per-document position reset.
    Keys: ``model.embed_tokens``, ``model.layers.N.*``, ``model.norm``, ``lm_head``
    (reference: models/qwen3/model.py:224-233)."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        self.config = config
        self.model = Decoder(config.text)
        if not config.text.tie_word_embeddings:
            self.lm_head = Linear(config.text.hidden_size, config.text.vocab_size)

    @property
    def decoder(self):
        return self.model


class _VLBackbone(nn.Module):
    def __init__(self, config: ModelConfig, with_vision: bool = True):
        super().__init__()
        self.language_model = Decoder(config.text)
        if config.vision is not None and with_vision:
            self.visual = VisionModel(config.vision)


class Qwen3VLForCausalLM(_CausalLMBase):
    """Qwen3-VL: ViT + DeepStack + interleaved-MRoPE decoder.
    Keys: ``model.language_model.*``, ``model.visual.*``, ``lm_head.weight``
    (reference: models/qwen3_vl/model.py:602-621)."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        self.config = config
        self.model = _VLBackbone(config)
        if not config.text.tie_word_embeddings:
            self.lm_head = Linear(config.text.hidden_size, config.text.vocab_size)

    @property
    def decoder(self):
        return self.model.language_model

    @property
    def visual(self):
        return getattr(self.model, "visual", None)


class Qwen3_5ForCausalLM(Qwen3VLForCausalLM):
    """Qwen3.5: hybrid Gated-DeltaNet / gated-attention decoder (dense or MoE MLP),
    same vision tower and key layout as Qwen3-VL (reference: models/qwen3_5/model.py:565-760).
    ``mtp.*`` tensors of a snapshot are ignored, as in the reference loader."""


MODEL_CLASSES = {"qwen3_text": Qwen3ForCausalLM, "qwen3_vl": Qwen3VLForCausalLM, "qwen3_5": Qwen3_5ForCausalLM}


def build_model(config: ModelConfig, dtype=torch.float32, device="cpu", init: bool = True, seed: int = 0):
    return MODEL_CLASSES[config.family].from_config(config, dtype=dtype, device=device, init=init, seed=seed)
