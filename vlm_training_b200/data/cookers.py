"""Cookers: crude webdataset samples (``jpg`` + ``json`` / ``txt``) → ``{"image", "messages"}`` in the
chat-template message format (reference: data/energon_dataloader.py:98-220).  Plain functions, usable
with or without megatron-energon."""
from __future__ import annotations

_ROLES = {"human": "user", "gpt": "assistant", "user": "user", "assistant": "assistant"}


def _img_then_text(caption: str) -> list[dict]:
    return [{"role": "user", "content": [{"type": "image"}]},
            {"role": "assistant", "content": [{"type": "text", "text": caption}]}]


def cook_llava_recap(sample: dict) -> dict:
    """LLaVA-recap: the caption is the second conversation turn."""
    return {"image": sample["jpg"], "messages": _img_then_text(sample["json"]["conversations"][1]["value"]),
            "__key__": sample.get("__key__", "")}


def cook_llava_imagenet(sample: dict, add_system_prompt: bool = True) -> dict:
    msgs = _img_then_text(sample["txt"])
    if not add_system_prompt:
        msgs.append({"role": "system", "content": [{"type": "text", "text": ""}]})
    return {"image": sample["jpg"], "messages": msgs, "__key__": sample.get("__key__", "")}


def cook_conversation(sample: dict, add_system_prompt: bool = True) -> dict:
    """Multi-turn instruct data (OneVision, captioning): roles mapped to user/assistant, the image goes
    where ``<image>`` appears or else into the first user turn."""
    msgs = []
    if not add_system_prompt:
        msgs.append({"role": "system", "content": [{"type": "text", "text": ""}]})
    placed = False
    for turn in sample["json"]["conversations"]:
        role = _ROLES.get(str(turn.get("from", turn.get("role", "user"))).lower(), "user")
        text = turn.get("value", turn.get("content", ""))
        content = []
        if "<image>" in text or (role == "user" and not placed):
            content.append({"type": "image"})
            text = text.replace("<image>", "").strip()
            placed = True
        if text:
            content.append({"type": "text", "text": text})
        if not content:
            content.append({"type": "text", "text": ""})
        msgs.append({"role": role, "content": content})
    return {"image": sample["jpg"], "messages": msgs, "__key__": sample.get("__key__", "")}


cook_onevision_instruct = cook_conversation
cook_captioning = cook_conversation

COOKERS = {"llava_recap": cook_llava_recap, "llava_imagenet": cook_llava_imagenet,
           "onevision_instruct": cook_onevision_instruct, "captioning": cook_captioning}
