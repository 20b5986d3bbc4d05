"""Packed-row (varlen) attention for stock Hugging Face model classes.

The reference carries a legacy module that monkey-patches the attention ``forward`` of HF's Qwen classes, ``create_causal_mask``
and the rope-index helpers so that a ``cu_seqlens`` tensor can travel where the attention mask goes (reference:
train/model_attention.py:1-361; its trainer no longer imports it).  The same capability needs no patched forwards here:
transformers keeps a registry of named attention functions and one of named mask functions.  :func:`register` adds
``"vlmt_varlen"`` to both: the mask function builds no dense mask, the attention function reads ``cu_seqlens`` from the
keyword arguments that the model's ``forward`` hands down to every layer and calls ``ops.attention_varlen`` (the tcgen05
kernel on a GPU, the plain PyTorch statement on CPU).  A batch is ONE packed row ``[1, T]`` whose position ids restart at
every document (:func:`packed_position_ids`)::

    from vlm_training_b200.utils import hf_varlen
    hf_varlen.enable(model)                       # any HF causal LM whose attention goes through the registry
    out = model(input_ids=ids[None], position_ids=hf_varlen.packed_position_ids(cu), cu_seqlens=cu)
"""
from __future__ import annotations

import torch

NAME = "vlmt_varlen"


def packed_position_ids(cu_seqlens: torch.Tensor) -> torch.Tensor:
    """``[1, T]`` positions that restart at 0 at every document boundary of ``cu_seqlens`` (``[n_docs + 1]``, starts at 0)."""
    cu = cu_seqlens.to(torch.long)
    total = int(cu[-1])
    starts = torch.repeat_interleave(cu[:-1], cu[1:] - cu[:-1], output_size=total)
    return (torch.arange(total, device=cu.device) - starts)[None]


def varlen_attention_forward(module, query, key, value, attention_mask=None, dropout: float = 0.0, scaling=None,
                             sliding_window=None, cu_seqlens=None, max_seqlen=None, **_unused):
    """The registry's calling convention: ``query [1, Hq, T, D]``, ``key`` / ``value`` ``[1, Hkv, T, D]`` ->
    ``([1, T, Hq, D], None)``.  ``cu_seqlens`` is required; dropout and sliding windows are not part of the packed kernels."""
    from .. import ops

    if cu_seqlens is None:
        raise ValueError(f"attention implementation {NAME!r} needs cu_seqlens=... in the model's forward call")
    if query.shape[0] != 1:
        raise ValueError("packed rows are one batch row [1, T]; got a batch of " + str(query.shape[0]))
    if dropout and module.training:
        raise ValueError("attention dropout is not supported by the packed attention kernels")
    if sliding_window is not None:
        raise ValueError("sliding-window attention is not supported by the packed attention kernels")
    q, k, v = (t[0].transpose(0, 1) for t in (query, key, value))   # [T, H, D]
    cu = cu_seqlens.to(device=q.device, dtype=torch.int32)
    if max_seqlen is None:
        max_seqlen = int((cu[1:] - cu[:-1]).max())
    out = ops.attention_varlen(q, k, v, cu, int(max_seqlen), causal=bool(getattr(module, "is_causal", True)), scale=scaling)
    return out[None], None


def _no_mask(*_args, **_kwargs):
    """Mask function of the registry: the document structure is in ``cu_seqlens``, no dense mask exists."""
    return None


def register(name: str = NAME) -> str:
    """Add the packed attention to transformers' registries (idempotent); returns the name to select it with."""
    from transformers import AttentionInterface, AttentionMaskInterface

    AttentionInterface.register(name, varlen_attention_forward)
    AttentionMaskInterface.register(name, _no_mask)
    return name


def enable(model, name: str = NAME):
    """Register the packed attention and select it for ``model`` (and the sub-configs of a multimodal model)."""
    register(name)
    if hasattr(model, "set_attn_implementation"):
        model.set_attn_implementation(name)
    else:
        model.config._attn_implementation = name
    return model
