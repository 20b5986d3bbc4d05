"""Streaming safetensors snapshot loader.

Supports sharded (``model.safetensors.index.json``) and single-file snapshots,
casts to the target dtype, raises on shape mismatch and on model keys that no
file provides (except a tied ``lm_head`` and prefixes the caller allows to be
missing), silently skips snapshot keys the model does not have such as
``mtp.*`` (reference: models/qwen3_vl/model.py:898-949, models/qwen3_5/utils.py:160-207).
"""
from __future__ import annotations

import json
import os

import torch


def snapshot_files(model_dir: str) -> list[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as fh:
            names = sorted(set(json.load(fh)["weight_map"].values()))
        return [os.path.join(model_dir, n) for n in names]
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(single):
        return [single]
    found = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not found:
        raise FileNotFoundError(f"no safetensors files in {model_dir}")
    return [os.path.join(model_dir, f) for f in found]


def load_snapshot_into(model, model_dir: str, dtype=None, allow_missing_prefixes=(), tied: bool = False,
                       key_map=None) -> dict:
    """Copy every tensor of the snapshot whose key the model's ``state_dict()`` has
    into the model, in place.  ``key_map`` optionally renames snapshot keys."""
    from safetensors import safe_open

    target = model.state_dict()  # HF-named views onto the (possibly fused) parameters
    loaded = set()
    for path in snapshot_files(model_dir):
        with safe_open(path, framework="pt", device="cpu") as fh:
            for key in fh.keys():
                name = key_map(key) if key_map else key
                if name is None or name not in target:
                    continue
                src = fh.get_tensor(key)
                dst = target[name]
                if tuple(src.shape) != tuple(dst.shape):
                    raise ValueError(f"shape mismatch for {name}: snapshot {tuple(src.shape)} vs model {tuple(dst.shape)}")
                with torch.no_grad():
                    dst.copy_(src.to(dst.dtype if dtype is None else dtype))
                loaded.add(name)
    missing = [k for k in target if k not in loaded
               and not (tied and k == "lm_head.weight")
               and not any(k.startswith(p) for p in allow_missing_prefixes)]
    if missing:
        raise RuntimeError(f"{len(missing)} model tensors not found in {model_dir}: {missing[:8]}...")
    return {"loaded": len(loaded), "missing_allowed": len(target) - len(loaded)}


def save_snapshot(model, config_dict: dict, out_dir: str, max_shard_bytes: int = 4 << 30):
    """Write the model as an HF-style safetensors snapshot (sharded + index)."""
    from safetensors.torch import save_file

    os.makedirs(out_dir, exist_ok=True)
    state = {k: v.detach().cpu().contiguous() for k, v in model.state_dict().items()}
    shards, cur, size = [], {}, 0
    for k, v in state.items():
        nb = v.numel() * v.element_size()
        if cur and size + nb > max_shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = v
        size += nb
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, shard in enumerate(shards):
        name = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, os.path.join(out_dir, name), metadata={"format": "pt"})
        weight_map.update({k: name for k in shard})
    if len(shards) > 1:
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as fh:
            json.dump({"metadata": {}, "weight_map": weight_map}, fh, indent=1)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(config_dict, fh, indent=1)
