"""Host-side batch pipeline: a background thread pulls rows from a dataset iterator, pins
them, and the training thread issues the host→device copies (non-blocking, from pinned
memory) and builds the :class:`BatchPlan` from the host metadata.

The reference pulls from an energon loader with two worker processes and then syncs with the
GPU several times per step to derive ``max_seqlen`` / position ids (reference:
train/train_qwen.py:403-442, models/qwen3_vl/model.py:674-679,765); here everything the
forward needs is already on the host when the batch arrives.
"""
from __future__ import annotations

import queue
import threading

import numpy as np
import torch

from ..models.causal_lm import BatchPlan
from ..models.vision import VisionPlan

_TENSOR_KEYS = ("input_ids", "labels", "cu_seqlens", "pixel_values", "image_grid_thw", "attention_mask", "mm_token_type_ids")


def make_dataset(data_cfg, training_cfg, model_cfg, dp_rank: int, dp_size: int, worker=(0, 1)):
    """The packed-row iterator of one data-parallel rank (module-level, so worker processes can build their own).
    ``worker = (w, n)``: this is worker ``w`` of ``n`` of that rank and reads / draws its own 1/n of the rank's rows."""
    w, n = worker
    if data_cfg.synthetic:
        from .synthetic import SyntheticDataset, spec_from_config

        spec = spec_from_config(data_cfg, model_cfg, seed=training_cfg.seed)
        return SyntheticDataset(spec, model_cfg, dp_rank=dp_rank, dp_size=dp_size, worker=worker)
    from .task_encoders import build_dataset

    return build_dataset(data_cfg, training_cfg, model_cfg, dp_rank=dp_rank * n + w, dp_size=dp_size * n)


def _worker_main(args, wid: int, n: int, out_q, stop):
    """Body of one data worker process: builds its dataset and feeds rows until told to stop.  Failures travel through
    the queue as exceptions; the end of the data as ``None``."""
    import traceback

    try:
        torch.set_num_threads(1)
        it = iter(make_dataset(*args, worker=(wid, n)))
        while not stop.is_set():
            item = next(it)
            while not stop.is_set():
                try:
                    out_q.put(item, timeout=0.2)
                    break
                except queue.Full:
                    continue
    except StopIteration:
        out_q.put(None)
    except BaseException as exc:  # noqa: BLE001 - everything is reported to the training process
        out_q.put(RuntimeError(f"data worker {wid} failed: {type(exc).__name__}: {exc}\n{traceback.format_exc()}"))


class WorkerPool:
    """Rows from ``n`` worker processes, taken in round-robin order (worker 0, 1, ..., n-1, 0, ...), so the sequence of
    rows is the same from run to run.  The reference reads through an energon loader with worker processes (reference:
    train/train_qwen.py:227-250); here a worker owns 1/n of the rank's samples (real data) or its own random stream
    (synthetic data).  A worker that raises is re-raised here; a worker that dies without a word is noticed by its exit
    code while its queue stays empty."""

    def __init__(self, args, n: int, depth: int = 2, start_method: str = "spawn"):
        import torch.multiprocessing as mp

        ctx = mp.get_context(start_method)
        self.n = int(n)
        self.stop = ctx.Event()
        self.queues = [ctx.Queue(maxsize=max(1, depth)) for _ in range(self.n)]
        self.procs = [ctx.Process(target=_worker_main, args=(args, w, self.n, self.queues[w], self.stop), daemon=True)
                      for w in range(self.n)]
        for p in self.procs:
            p.start()
        self.done = [False] * self.n
        self.turn = 0

    def __iter__(self):
        return self

    def __next__(self):
        while not all(self.done):
            w = self.turn
            if self.done[w]:
                self.turn = (w + 1) % self.n
                continue
            try:
                item = self.queues[w].get(timeout=0.5)
            except queue.Empty:
                if not self.procs[w].is_alive() and self.queues[w].empty():
                    self.close()
                    raise RuntimeError(f"data worker {w} exited with code {self.procs[w].exitcode} without reporting")
                continue
            except (ConnectionError, EOFError, OSError) as exc:
                # a queued row whose tensors were still owned by the worker: they cannot be received once it is gone
                if not self.procs[w].is_alive():
                    code = self.procs[w].exitcode
                    self.close()
                    raise RuntimeError(f"data worker {w} exited with code {code} without reporting") from exc
                raise
            self.turn = (w + 1) % self.n
            if item is None:
                self.done[w] = True
                continue
            if isinstance(item, Exception):
                self.close()
                raise item
            return item
        raise StopIteration

    def close(self):
        self.stop.set()
        for q_ in self.queues:
            try:
                while True:
                    q_.get_nowait()
            except (queue.Empty, OSError, ValueError, EOFError):
                # empty, closed, or a queued row whose tensor storage belonged to a worker that has already left
                pass
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
                p.join(timeout=5)


class PrefetchLoader:
    """``transfer``: optional ``batch -> kwargs`` callable (see :func:`to_device`) run by the worker thread on its own
    CUDA stream, so the host→device copies and the plan construction of step n+1 overlap step n; ``__next__`` then
    returns the device-side kwargs and makes the consumer's stream wait for the copies."""

    def __init__(self, dataset, depth: int = 2, pin: bool = True, transfer=None, device=None):
        self.source = dataset
        self.dataset = iter(dataset)
        self.pin = pin and torch.cuda.is_available()
        self.transfer = transfer
        self.device = device
        self.stream = torch.cuda.Stream(device=device) if (transfer is not None and device is not None
                                                            and torch.device(device).type == "cuda") else None
        self.q: queue.Queue = queue.Queue(maxsize=depth)
        self._stop = False
        self.thread = threading.Thread(target=self._work, daemon=True)
        self.thread.start()

    def _put(self, item) -> bool:
        while not self._stop:
            try:
                self.q.put(item, timeout=0.1)
                return True
            except queue.Full:
                continue
        return False

    def _work(self):
        try:
            while not self._stop:
                batch = next(self.dataset)
                if self.pin:
                    for k in _TENSOR_KEYS:
                        if k in batch and torch.is_tensor(batch[k]):
                            batch[k] = batch[k].pin_memory()
                if self.transfer is not None:
                    meta = {"n_tokens": int(batch["input_ids"].numel()), "n_label": int((batch["labels"] != -100).sum()),
                            "n_docs": int(batch["cu_seqlens"].numel()) - 1, "h2d_bytes": batch_nbytes(batch)}
                    if self.stream is not None:
                        with torch.cuda.stream(self.stream):
                            kwargs = self.transfer(batch)
                            ev = torch.cuda.Event()
                            ev.record(self.stream)
                    else:
                        kwargs, ev = self.transfer(batch), None
                    batch = {"kwargs": kwargs, "event": ev, "meta": meta, "host_batch": batch}
                if not self._put(batch):
                    return
        except StopIteration:
            self._put(None)
        except Exception as exc:  # surface worker failures in the training thread
            self._put(exc)

    def __iter__(self):
        return self

    def __next__(self):
        item = self.q.get()
        if item is None:
            raise StopIteration
        if isinstance(item, Exception):
            raise item
        if self.transfer is not None and item.get("event") is not None:
            cur = torch.cuda.current_stream()
            cur.wait_event(item["event"])
            for t in _tensors_of(item["kwargs"]):
                t.record_stream(cur)  # allocated on the loader's stream, consumed on the training stream
        return item

    def close(self):
        """Stop the worker and wait for it, so no thread touches CUDA (pinned allocations) during interpreter exit."""
        self._stop = True
        if hasattr(self.source, "close"):
            self.source.close()
        try:
            while True:
                self.q.get_nowait()
        except queue.Empty:
            pass
        if self.thread.is_alive() and threading.current_thread() is not self.thread:
            self.thread.join(timeout=30)


def _tensors_of(obj):
    if torch.is_tensor(obj):
        if obj.is_cuda:
            yield obj
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from _tensors_of(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _tensors_of(v)
    elif hasattr(obj, "__dataclass_fields__"):
        for name in obj.__dataclass_fields__:
            yield from _tensors_of(getattr(obj, name))


def batch_nbytes(batch: dict) -> int:
    """Bytes of one batch that cross host→device (tensors + host-built plan tables)."""
    n = 0
    for k in ("input_ids", "labels", "cu_seqlens", "pixel_values", "image_grid_thw"):
        if k in batch and torch.is_tensor(batch[k]):
            n += batch[k].numel() * batch[k].element_size()
    for v in batch.get("host", {}).values():
        if isinstance(v, np.ndarray):
            n += v.nbytes
    return n


def to_device(batch: dict, cfg, device, pixel_dtype=torch.bfloat16) -> dict:
    """Copy one batch to ``device`` and assemble the model call's keyword arguments.
    As in the reference trainer, ``attention_mask`` becomes ``cu_seqlens`` (train/train_qwen.py:420)."""
    nb = device.type == "cuda"
    ids = batch["input_ids"].to(device, non_blocking=nb)
    labels = batch["labels"].to(device, non_blocking=nb)
    cu = batch["cu_seqlens"].to(device=device, dtype=torch.int32, non_blocking=nb)
    host = batch.get("host")
    grids = batch.get("image_grid_thw")
    kwargs = {"input_ids": ids, "labels": labels, "attention_mask": cu}
    if host is None:
        plan = BatchPlan.build(cfg, batch["input_ids"], batch["cu_seqlens"], grids if "pixel_values" in batch else None, device)
    else:
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=dt, non_blocking=nb)
        plan = BatchPlan(cu, int(host["max_seqlen"]), t(host["position_ids"], torch.int64))
        plan.extras["cu_host"] = batch["cu_seqlens"].tolist()
        if "seq_idx" in host:
            plan.seq_idx = t(host["seq_idx"], torch.int32)
        if "image_rows" in host:
            plan.image_rows = t(host["image_rows"], torch.int64)
            plan.image_rows_host = host["image_rows"]
            plan.vision = VisionPlan.build(grids.tolist(), cfg.vision, device)
    if "pixel_values" in batch:
        kwargs["pixel_values"] = batch["pixel_values"].to(device=device, dtype=pixel_dtype, non_blocking=nb)
        kwargs["image_grid_thw"] = grids
    kwargs["batch_plan"] = plan
    return kwargs
