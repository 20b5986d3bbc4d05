"""Task encoders: raw samples → the packed-row batch contract.

Three encoders, selected as in the reference factory (reference: data/task_encoder_factory.py:24-41):
``text_dataset`` → :class:`TextEncoder`; ``batch_size > 0`` → :class:`SingleBatchEncoder` (a fixed
number of samples per row); ``batch_size == 0`` → :class:`PackedBatchEncoder` (online packing of a
buffer of ``packing_buffer_size`` samples).  The encoders are plain Python: ``encode_sample`` works
on one cooked sample, ``rows(iterable)`` yields batches.  When ``megatron.energon`` is importable,
``build_dataset`` reads ``data.data_path`` through it (crude webdatasets, rank-sharded, energon's worker
processes; every item is normalised, cooked by the cooker that ``data.cooker`` names or the sample's fields
imply, and then encoded); otherwise it accepts a ``.jsonl`` / ``.txt`` file of documents for text training
and raises a clear error for multimodal paths.
"""
from __future__ import annotations

import json
import os
import random

import torch

from ..models.config import ModelConfig
from . import cookers
from .packing import assistant_label_mask, collate_row, select_bins
from .synthetic import host_plan


def _with_plan(batch: dict, cfg: ModelConfig) -> dict:
    np_batch = {"input_ids": batch["input_ids"].numpy(), "cu_seqlens": batch["cu_seqlens"].numpy()}
    if "image_grid_thw" in batch:
        np_batch["image_grid_thw"] = batch["image_grid_thw"].numpy()
    batch["host"] = host_plan(np_batch, cfg)
    return batch


class TextEncoder:
    """Tokenise documents, concatenate, pad to the row length; labels = ids with pads masked and, unlike the
    reference (data/energon_dataloader.py:82-83), the first token of each document masked so one document is
    never trained to predict the next."""

    def __init__(self, tokenizer, max_len: int, samples_per_row: int = 0):
        self.tokenizer, self.max_length, self.samples_per_row = tokenizer, int(max_len), samples_per_row

    def encode_sample(self, sample) -> dict:
        text = sample["text"] if isinstance(sample, dict) else getattr(sample, "text", sample)
        ids = self.tokenizer(text=text, return_tensors="pt", padding=False, truncation=True, max_length=self.max_length,
                             add_special_tokens=True)["input_ids"][0]
        labels = ids.clone()
        labels[0] = -100
        return {"input_ids": ids, "labels": labels}

    def rows(self, samples, cfg: ModelConfig):
        cur, used = [], 0
        for s in samples:
            e = self.encode_sample(s)
            n = int(e["input_ids"].numel())
            full = used + n > self.max_length or (self.samples_per_row and len(cur) >= self.samples_per_row)
            if cur and full:
                yield _with_plan(collate_row(cur, self.max_length, self.tokenizer.pad_token_id), cfg)
                cur, used = [], 0
            cur.append(e)
            used += n
        if cur:
            yield _with_plan(collate_row(cur, self.max_length, self.tokenizer.pad_token_id), cfg)


class _VLMEncoder:
    def __init__(self, processor, max_seq_len: int, cooker=cookers.cook_captioning):
        self.processor, self.tokenizer = processor, processor.tokenizer
        self.max_length = int(max_seq_len)
        self.cooker = cooker
        self.assistant_token = self.tokenizer.encode("assistant")[0]
        self.eos_token = self.tokenizer.eos_token_id

    def encode_sample(self, sample: dict) -> dict:
        cooked = sample if "messages" in sample else self.cooker(sample)
        text = self.processor.apply_chat_template(conversation=cooked["messages"], tokenize=False, add_generation_prompt=False)
        images = [cooked["image"]] if cooked.get("image") is not None else None
        enc = self.processor(text=[text], images=images, padding=False, return_tensors="pt")
        ids = enc["input_ids"][0]
        out = {"input_ids": ids, "attention_mask": enc["attention_mask"][0],
               "labels": assistant_label_mask(ids, self.assistant_token, self.eos_token)}
        if enc.get("pixel_values") is not None:
            out["pixel_values"], out["image_grid_thw"] = enc["pixel_values"], enc["image_grid_thw"]
        if enc.get("mm_token_type_ids") is not None:
            out["mm_token_type_ids"] = enc["mm_token_type_ids"][0]
        return out


class SingleBatchEncoder(_VLMEncoder):
    """A fixed number of samples per row, no packing decisions (reference: data/energon_dataloader.py:234-337)."""

    def __init__(self, processor, max_seq_len: int, batch_size: int, **kw):
        super().__init__(processor, max_seq_len, **kw)
        self.batch_size = batch_size

    def rows(self, samples, cfg: ModelConfig):
        cur = []
        for s in samples:
            cur.append(self.encode_sample(s))
            if len(cur) == self.batch_size:
                yield _with_plan(collate_row(cur, self.max_length, self.tokenizer.pad_token_id), cfg)
                cur = []


class PackedBatchEncoder(_VLMEncoder):
    """Online packing: buffer ``packing_buffer_size`` encoded samples, bin them first-fit by decreasing
    length, emit one row per bin (reference: data/energon_dataloader.py:339-464)."""

    def __init__(self, processor, max_seq_len: int, packing_buffer_size: int, seed: int = 0, **kw):
        super().__init__(processor, max_seq_len, **kw)
        self.buffer_size = max(1, packing_buffer_size)
        self.rng = random.Random(seed)

    def rows(self, samples, cfg: ModelConfig):
        buf = []

        def flush():
            for b in select_bins([int(e["input_ids"].numel()) for e in buf], self.max_length, self.rng):
                yield _with_plan(collate_row([buf[i] for i in b], self.max_length, self.tokenizer.pad_token_id), cfg)

        for s in samples:
            buf.append(self.encode_sample(s))
            if len(buf) >= self.buffer_size:
                yield from flush()
                buf = []
        if buf:
            yield from flush()


def build_task_encoder(data_args, tokenizer, processor):
    """→ ``(encoder, extra_kwargs)`` with the reference's dispatch rule."""
    seq = int(data_args.seq_len)
    if data_args.text_dataset:
        return TextEncoder(tokenizer, seq, samples_per_row=data_args.max_samples_per_sequence), {}
    if data_args.batch_size > 0:
        return SingleBatchEncoder(processor, seq, data_args.batch_size), {}
    return PackedBatchEncoder(processor, seq, data_args.packing_buffer_size), {"packing_buffer_size": data_args.packing_buffer_size}


def _read_text_file(path: str, rank: int, world: int):
    with open(path) as fh:
        for i, line in enumerate(fh):
            if i % world != rank:
                continue
            line = line.strip()
            if not line:
                continue
            yield json.loads(line) if path.endswith(".jsonl") else {"text": line}


def pick_cooker(sample: dict, name: str = "auto"):
    """The cooker for a crude sample: by name (``data.cooker``), or from the sample's fields: ``json`` with a
    ``conversations`` list → the conversation cooker, ``txt`` → image + caption."""
    if name != "auto":
        return cookers.COOKERS[name]
    js = sample.get("json")
    if isinstance(js, (bytes, str)):
        js = json.loads(js)
    if isinstance(js, dict) and "conversations" in js:
        return cookers.cook_conversation
    if "txt" in sample:
        return cookers.cook_llava_imagenet
    raise KeyError(f"cannot choose a cooker for a sample with fields {sorted(sample)}; set data.cooker")


def normalise_crude(item) -> dict:
    """One loader item → a plain crude-sample dict: unwraps the batch of one that ``batch_size=1`` produces, turns
    sample objects into dicts, decodes ``json`` / ``txt`` bytes and opens ``jpg`` / ``png`` bytes with PIL (decoding
    here, not in the HF processor, keeps the pixel scaling single as in the reference, data/energon_dataloader.py:242-247)."""
    if isinstance(item, (list, tuple)) and len(item) == 1:
        item = item[0]
    if not isinstance(item, dict):
        item = {k: getattr(item, k) for k in dir(item) if not k.startswith("_") and not callable(getattr(item, k))}
    out = dict(item)
    for k in ("json", "txt"):
        v = out.get(k)
        if isinstance(v, bytes):
            v = v.decode("utf-8")
        if k == "json" and isinstance(v, str):
            v = json.loads(v)
        if v is not None:
            out[k] = v
    for k in ("jpg", "jpeg", "png"):
        v = out.get(k)
        if isinstance(v, bytes):
            import io

            from PIL import Image

            v = Image.open(io.BytesIO(v)).convert("RGB")
        if v is not None:
            out["jpg"] = v
    return out


def _energon_samples(path: str, data_args, rank: int, world: int):
    """Cooked samples from an energon (crude webdataset) path, sharded over the data-parallel ranks; energon's own
    loader runs ``data.num_workers`` worker processes (reference: train/train_qwen.py:227-250).  Text datasets pass
    through uncooked."""
    from megatron.energon import WorkerConfig, get_loader, get_train_dataset  # optional dependency

    wc = WorkerConfig(rank=rank, world_size=world, num_workers=data_args.num_workers)
    ds = get_train_dataset(path, batch_size=1, shuffle_buffer_size=data_args.shuffle_buffer_size,
                           max_samples_per_sequence=data_args.max_samples_per_sequence, worker_config=wc, repeat=False)
    cooker = None
    for item in get_loader(ds):
        if data_args.text_dataset:
            yield item[0] if isinstance(item, (list, tuple)) and len(item) == 1 else item
            continue
        crude = normalise_crude(item)
        if "messages" in crude:
            yield crude
            continue
        if cooker is None:
            cooker = pick_cooker(crude, getattr(data_args, "cooker", "auto"))
        yield cooker(crude)


def build_dataset(data_args, training_args, cfg: ModelConfig, dp_rank: int, dp_size: int):
    """Iterator of packed-row batches for real data.  Tensor-parallel peers pass the same ``dp_rank`` and
    therefore read identical rows (reference: train/train_qwen.py:227-232)."""
    import transformers

    tok = transformers.AutoTokenizer.from_pretrained(training_args.model_dir, model_max_length=int(data_args.seq_len),
                                                     padding_side="right")
    proc = None
    if not data_args.text_dataset:
        proc = transformers.AutoProcessor.from_pretrained(training_args.model_dir, max_pixels=1048576)
    enc, _ = build_task_encoder(data_args, tok, proc)
    path = data_args.data_path
    if os.path.isfile(path) and path.endswith((".jsonl", ".txt")):
        samples = _read_text_file(path, dp_rank, dp_size)
    else:
        try:
            samples = _energon_samples(path, data_args, dp_rank, dp_size)
        except ImportError as exc:
            raise ImportError("data.data_path is not a .jsonl/.txt file and megatron-energon is not installed; "
                              "install it to read energon webdatasets, or set data.synthetic") from exc
    return enc.rows(samples, cfg)
