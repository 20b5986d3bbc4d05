"""Terminal chat with a trained snapshot (greedy decoding, optional image).

    python -m vlm_training_b200.utils.chat --model_dir SNAPSHOT [--image path_or_url] [--max_new_tokens 256]

The reference drives HF ``generate`` (reference: utils/chat.py:1-75); this one runs the native model and
re-evaluates the full prefix for every new token (no KV cache, as the reference's generation tests do).
"""
from __future__ import annotations

import argparse

import torch


@torch.no_grad()
def greedy_generate(model, input_ids, max_new_tokens: int, eos_token_id: int | None = None, **mm):
    ids = input_ids.reshape(1, -1)
    for _ in range(max_new_tokens):
        logits = model(ids, **mm)
        nxt = logits[0, -1].argmax().reshape(1, 1)
        ids = torch.cat((ids, nxt), 1)
        if eos_token_id is not None and int(nxt) == eos_token_id:
            break
    return ids


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_dir", required=True)
    ap.add_argument("--image", default=None)
    ap.add_argument("--max_new_tokens", type=int, default=256)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    import transformers

    from ..models import MODEL_CLASSES, ModelConfig

    cfg = ModelConfig.from_json(f"{a.model_dir}/config.json")
    dtype = torch.bfloat16 if a.device == "cuda" else torch.float32
    model, _ = MODEL_CLASSES[cfg.family].from_pretrained(a.model_dir, dtype=dtype, device=a.device)
    model.eval()
    proc = transformers.AutoProcessor.from_pretrained(a.model_dir) if cfg.vision is not None else None
    tok = proc.tokenizer if proc is not None else transformers.AutoTokenizer.from_pretrained(a.model_dir)
    image = None
    if a.image:
        from PIL import Image

        if a.image.startswith("http"):
            import io
            import urllib.request

            image = Image.open(io.BytesIO(urllib.request.urlopen(a.image).read())).convert("RGB")
        else:
            image = Image.open(a.image).convert("RGB")
    history = []
    while True:
        try:
            text = input("user> ").strip()
        except EOFError:
            break
        if text in ("", "exit", "quit"):
            break
        content = [{"type": "text", "text": text}]
        if image is not None and not history:
            content.insert(0, {"type": "image"})
        history.append({"role": "user", "content": content})
        if proc is not None:
            prompt = proc.apply_chat_template(history, tokenize=False, add_generation_prompt=True)
            enc = proc(text=[prompt], images=[image] if image is not None else None, return_tensors="pt")
        else:
            prompt = tok.apply_chat_template(history, tokenize=False, add_generation_prompt=True)
            enc = tok(prompt, return_tensors="pt")
        mm = {}
        if enc.get("pixel_values") is not None:
            mm = {"pixel_values": enc["pixel_values"].to(a.device, dtype), "image_grid_thw": enc["image_grid_thw"]}
        out = greedy_generate(model, enc["input_ids"].to(a.device), a.max_new_tokens, tok.eos_token_id, **mm)
        reply = tok.decode(out[0, enc["input_ids"].shape[1]:], skip_special_tokens=True)
        print(f"assistant> {reply}")
        history.append({"role": "assistant", "content": [{"type": "text", "text": reply}]})


if __name__ == "__main__":
    main()
