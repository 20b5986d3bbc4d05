"""DCP checkpoints → HF safetensors snapshots.

    python -m vlm_training_b200.utils.convert --ckpt_dir OUT --base_model HF_SNAPSHOT_OR_PRESET [--step N] [--out models]

Converts every ``checkpoint-step-*`` under ``--ckpt_dir`` (or one ``--step``) into
``<out>/step-N`` (``model*.safetensors`` + ``config.json``) — the batch converter of the
reference (reference: utils/convertion_script.py:24-117).  The ``model.`` entry prefix of the
DCP state dict is stripped, any ``._orig_mod`` / ``_checkpoint_wrapped_module.`` segments from
wrappers are removed, and at least 95 % of the model's keys must be found in the checkpoint.
"""
from __future__ import annotations

import argparse
import json
import os
import re

import torch


def _clean(key: str) -> str:
    key = key[len("model."):] if key.startswith("model.") else key
    return key.replace("._orig_mod", "").replace("_checkpoint_wrapped_module.", "")


def load_model_from_dcp(ckpt_path: str, model) -> tuple[int, int]:
    """Fill ``model`` (CPU) from the ``model`` entry of a DCP checkpoint. Returns (loaded, total)."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader

    meta = FileSystemReader(ckpt_path).read_metadata()
    available = {k: v for k, v in meta.state_dict_metadata.items() if k.startswith("model.")}
    target = model.state_dict()
    by_clean = {_clean(k): k for k in available}
    bufs, names = {}, {}
    for name, t in target.items():
        src = by_clean.get(name)
        if src is None:
            continue
        bufs[src] = torch.empty(tuple(available[src].size), dtype=t.dtype)
        names[src] = name
    if len(bufs) < 0.95 * len(target):
        raise RuntimeError(f"only {len(bufs)}/{len(target)} model tensors found in {ckpt_path}")
    dcp.load(bufs, checkpoint_id=ckpt_path, no_dist=True)
    with torch.no_grad():
        for src, name in names.items():
            target[name].copy_(bufs[src])
    return len(bufs), len(target)


def convert(ckpt_dir: str, base_model: str, out_dir: str, step: int | None = None, dtype=torch.bfloat16):
    from ..models import MODEL_CLASSES, ModelConfig
    from ..models.loader import save_snapshot

    if os.path.isdir(base_model):
        cfg = ModelConfig.from_json(os.path.join(base_model, "config.json"))
        with open(os.path.join(base_model, "config.json")) as fh:
            cfg_dict = json.load(fh)
    else:
        cfg = ModelConfig.preset(base_model)
        cfg_dict = cfg.to_dict()
    model = MODEL_CLASSES[cfg.family].from_config(cfg, dtype=dtype, device="cpu", init=False)
    done = []
    for name in sorted(os.listdir(ckpt_dir)):
        m = re.search(r"checkpoint-step-(\d+)$", name)
        if not m or (step is not None and int(m.group(1)) != step):
            continue
        path = os.path.join(ckpt_dir, name)
        n, total = load_model_from_dcp(path, model)
        dst = os.path.join(out_dir, f"step-{m.group(1)}")
        save_snapshot(model, cfg_dict, dst)
        print(f"{path} -> {dst} ({n}/{total} tensors)")
        done.append(dst)
    if not done:
        raise FileNotFoundError(f"no checkpoint-step-* directories under {ckpt_dir}")
    return done


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ckpt_dir", required=True)
    ap.add_argument("--base_model", required=True, help="HF snapshot directory (for config.json) or a preset name")
    ap.add_argument("--out", default="models")
    ap.add_argument("--step", type=int, default=None)
    a = ap.parse_args(argv)
    convert(a.ckpt_dir, a.base_model, a.out, a.step)


if __name__ == "__main__":
    main()
