"""Perplexity evaluation on a held-out stream.

    torchrun --nproc-per-node N -m vlm_training_b200.eval.val --model_dir SNAPSHOT --data_path val.jsonl [--seq_len 4096]

Mean next-token loss over all ranks (two all-reduces: loss sum and token count) and ``exp`` of it
(reference: eval/val.py:1-113, which uses the HF model class + torch DDP; here the native model runs on each
rank's shard of the data with no gradient synchronisation to set up).
"""
from __future__ import annotations

import argparse
import math

import torch
import torch.distributed as dist


@torch.no_grad()
def evaluate(model, rows, device, max_rows: int | None = None) -> tuple[float, int]:
    from ..data.loader import to_device

    loss_sum, n_tok = 0.0, 0
    for i, batch in enumerate(rows):
        if max_rows is not None and i >= max_rows:
            break
        kw = to_device(batch, model.config, device, pixel_dtype=next(model.parameters()).dtype)
        out = model(**kw)
        loss_sum += float(out.loss_sum)
        n_tok += int(out.n_valid)
    return loss_sum, n_tok


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_dir", required=True)
    ap.add_argument("--data_path", required=True)
    ap.add_argument("--seq_len", type=int, default=4096)
    ap.add_argument("--text_dataset", action="store_true", default=True)
    ap.add_argument("--max_rows", type=int, default=None)
    a = ap.parse_args(argv)
    from ..config import Config
    from ..data.task_encoders import build_dataset
    from ..models import MODEL_CLASSES, ModelConfig
    from ..parallel.mesh import init_distributed

    rank, world, device = init_distributed()
    cfg = ModelConfig.from_json(f"{a.model_dir}/config.json")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model, _ = MODEL_CLASSES[cfg.family].from_pretrained(a.model_dir, dtype=dtype, device=device)
    model.eval()
    c = Config()
    c.data.data_path, c.data.seq_len, c.data.text_dataset = a.data_path, a.seq_len, a.text_dataset
    c.training.model_dir = a.model_dir
    rows = build_dataset(c.data, c.training, cfg, dp_rank=rank, dp_size=world)
    loss_sum, n_tok = evaluate(model, rows, device, a.max_rows)
    t = torch.tensor([loss_sum, float(n_tok)], dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
    if dist.is_initialized():
        dist.all_reduce(t)
    loss = float(t[0] / max(t[1], 1))
    if rank == 0:
        print(f"tokens {int(t[1])}  loss {loss:.4f}  ppl {math.exp(loss):.3f}")
    if dist.is_initialized():
        dist.destroy_process_group()
    return loss


if __name__ == "__main__":
    main()
