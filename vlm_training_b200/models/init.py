"""Weight initialisation recipes.

``init_normal_`` is the benchmark recipe ("all weights normal(0, 0.02)", norms at
their identity value).  ``init_qwen35_`` and ``init_qwen3vl_`` restate the two
``random_init`` recipes of the reference trainer (reference: train/utils.py:35-86);
instead of one broadcast per parameter they draw from a seeded generator that
every rank shares, so all ranks produce identical weights without communication.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


_CUDA_GENS = {}


def _normal_(p: torch.Tensor, std: float, gen: torch.Generator):
    with torch.no_grad():
        if p.is_cuda:
            # large models are initialised in place on the GPU; the device generator is seeded from the
            # host generator so every rank (same seed, same GPU type) draws the same values
            key = (p.device, id(gen))
            if key not in _CUDA_GENS:
                g = torch.Generator(device=p.device)
                g.manual_seed(int(torch.randint(0, 2 ** 31 - 1, (1,), generator=gen)))
                _CUDA_GENS[key] = g
            p.normal_(0.0, std, generator=_CUDA_GENS[key])
            return
        # CPU: draw in fp32 chunks so the values do not depend on the parameter dtype
        chunk = 1 << 24
        flat = p.view(-1)
        for s in range(0, flat.numel(), chunk):
            n = min(chunk, flat.numel() - s)
            flat[s:s + n].copy_(torch.empty(n, dtype=torch.float32).normal_(0.0, std, generator=gen))


def init_normal_(model: nn.Module, std: float = 0.02, seed: int = 0, only_uninitialised: bool = False):
    from .layers import GatedRMSNorm, RMSNorm

    gen = _gen(None, seed)
    with torch.no_grad():
        for name, mod in model.named_modules():
            if isinstance(mod, RMSNorm):
                mod.weight.fill_(0.0 if mod.offset else 1.0)
            elif isinstance(mod, GatedRMSNorm):
                mod.weight.fill_(1.0)
            elif isinstance(mod, nn.LayerNorm):
                mod.weight.fill_(1.0)
                mod.bias.zero_()
        for name, p in model.named_parameters():
            leaf = name.rsplit(".", 1)[-1]
            owner = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
            if isinstance(owner, (RMSNorm, GatedRMSNorm, nn.LayerNorm)):
                continue
            if leaf == "bias":
                p.zero_()
            elif leaf == "A_log":
                p.zero_()
            elif leaf == "dt_bias":
                p.fill_(1.0)
            else:
                _normal_(p, std, gen)
    return model


def init_qwen35_(model: nn.Module, seed: int = 42):
    """N(0, 0.02) for every Linear/Embedding weight of the decoder and the merger,
    biases 0, every norm weight 1 (this also overwrites the zero-init offset
    norms with ones, as the reference does), then ``o_proj``/``down_proj`` ~
    N(0, 0.02/sqrt(2L)) (reference: train/utils.py:35-72)."""
    from .layers import GatedRMSNorm, RMSNorm

    gen = _gen(None, seed)
    n_layers = model.config.text.num_hidden_layers
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "visual." in name and "merger" not in name:
                continue
            owner = model.get_submodule(name.rsplit(".", 1)[0])
            leaf = name.rsplit(".", 1)[-1]
            if isinstance(owner, (RMSNorm, GatedRMSNorm, nn.LayerNorm)):
                if leaf == "weight":
                    p.fill_(1.0)
                else:
                    p.zero_()
            elif leaf == "bias":
                p.zero_()
            elif leaf in ("A_log", "dt_bias"):
                continue
            elif name.endswith("o_proj.weight") or name.endswith("down_proj.weight") or name.endswith("experts.down_proj"):
                _normal_(p, 0.02 / math.sqrt(2 * n_layers), gen)
            else:
                _normal_(p, 0.02, gen)
    return model


def init_qwen3vl_(model: nn.Module, seed: int = 42):
    """Xavier-uniform on the merger and the DeepStack mergers only
    (reference: train/utils.py:74-86)."""
    gen = _gen(None, seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "visual.merger" not in name and "visual.deepstack_merger_list" not in name:
                continue
            if p.dim() < 2:
                if name.endswith("bias"):
                    p.zero_()
                continue
            fan_out, fan_in = p.shape[0], p.shape[1]
            bound = math.sqrt(6.0 / (fan_in + fan_out))
            p.copy_((torch.rand(p.shape, generator=gen, dtype=torch.float32) * 2 - 1) * bound)
    return model
