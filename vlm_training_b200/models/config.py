"""Architecture descriptions for the three model families.

One ``TextConfig`` covers the Qwen3, Qwen3-VL and Qwen3.5 (dense and MoE)
decoders; the family-specific behaviour is selected by fields, not by
subclasses.  ``from_hf_dict`` reads the ``config.json`` fields the reference
loaders consume (reference: models/qwen3/model.py:38-70,
models/qwen3_vl/model.py:108-153, models/qwen3_5/config.py:58-110);
``preset`` builds the shapes named by the benchmark configurations when no
snapshot exists.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path


@dataclass
class TextConfig:
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    max_position_embeddings: int = 262144
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    # rotary: None → plain 1-D RoPE (text Qwen3); a 3-list → interleaved MRoPE
    mrope_section: list[int] | None = None
    partial_rotary_factor: float = 1.0
    # Qwen3.5 switches
    offset_norm: bool = False  # RMSNorm weight stored as (w - 1)
    attn_output_gate: bool = False  # q_proj emits [q | gate] per head
    layer_types: list[str] | None = None  # "full_attention" | "linear_attention"
    full_attention_interval: int = 4
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 16
    # MoE (0 experts → dense SwiGLU MLP)
    num_experts: int = 0
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512
    norm_topk_prob: bool = True
    # DSA sparse attention on full-attention layers
    dsa: bool = False
    dsa_topk: int = 2048
    dsa_index_heads: int = 4
    dsa_index_dim: int = 64

    @property
    def rope_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    def layer_type(self, i: int) -> str:
        if self.layer_types is not None:
            return self.layer_types[i]
        return "full_attention"

    @property
    def is_hybrid(self) -> bool:
        return self.layer_types is not None and any(t == "linear_attention" for t in self.layer_types)


@dataclass
class VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    num_position_embeddings: int = 2304
    out_hidden_size: int = 4096
    hidden_act: str = "gelu_pytorch_tanh"
    deepstack_visual_indexes: list[int] = field(default_factory=lambda: [8, 16, 24])

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


@dataclass
class ModelConfig:
    family: str = "qwen3_text"  # "qwen3_text" | "qwen3_vl" | "qwen3_5"
    text: TextConfig = field(default_factory=TextConfig)
    vision: VisionConfig | None = None
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    vision_end_token_id: int = 151653
    torch_dtype: str = "bfloat16"

    def to_dict(self) -> dict:
        return asdict(self)

    # ------------------------------------------------------------------ HF json
    @classmethod
    def from_json(cls, path: str | Path) -> "ModelConfig":
        with open(path, "r") as fh:
            return cls.from_hf_dict(json.load(fh))

    @classmethod
    def from_hf_dict(cls, raw: dict) -> "ModelConfig":
        mt = (raw.get("model_type") or "").lower()
        if "text_config" not in raw:
            return cls(family="qwen3_text", text=_text_from_hf(raw, raw, "qwen3_text"),
                       torch_dtype=raw.get("torch_dtype") or raw.get("dtype") or "bfloat16")
        family = "qwen3_5" if "qwen3_5" in mt or "layer_types" in raw["text_config"] else "qwen3_vl"
        text = _text_from_hf(raw["text_config"], raw, family)
        vc = dict(raw["vision_config"])
        vision = VisionConfig(
            depth=vc["depth"], hidden_size=vc["hidden_size"], intermediate_size=vc["intermediate_size"],
            num_heads=vc["num_heads"], in_channels=vc.get("in_channels", 3), patch_size=vc["patch_size"],
            temporal_patch_size=vc["temporal_patch_size"], spatial_merge_size=vc["spatial_merge_size"],
            num_position_embeddings=vc["num_position_embeddings"], out_hidden_size=vc["out_hidden_size"],
            hidden_act=vc.get("hidden_act", "gelu_pytorch_tanh"),
            # HF Qwen3.5 vision configs carry no deepstack list: none is used
            deepstack_visual_indexes=list(vc.get("deepstack_visual_indexes") or []),
        )
        return cls(family=family, text=text, vision=vision,
                   image_token_id=raw.get("image_token_id", 151655), video_token_id=raw.get("video_token_id", 151656),
                   vision_start_token_id=raw.get("vision_start_token_id", 151652),
                   vision_end_token_id=raw.get("vision_end_token_id", 151653),
                   torch_dtype=raw.get("torch_dtype") or raw["text_config"].get("dtype") or "bfloat16")

    # ------------------------------------------------------------------ presets
    @classmethod
    def preset(cls, name: str, **overrides) -> "ModelConfig":
        name = name.lower()
        if name not in _PRESETS:
            raise ValueError(f"unknown preset {name!r}; have {sorted(_PRESETS)}")
        cfg = _PRESETS[name]()
        for k, v in overrides.items():
            if hasattr(cfg.text, k):
                setattr(cfg.text, k, v)
            elif cfg.vision is not None and hasattr(cfg.vision, k):
                setattr(cfg.vision, k, v)
            else:
                raise ValueError(f"unknown override {k}")
        return cfg


def _text_from_hf(tc: dict, root: dict, family: str) -> TextConfig:
    rope = tc.get("rope_parameters") or tc.get("rope_scaling") or {}
    heads = tc["num_attention_heads"]
    cfg = TextConfig(
        vocab_size=tc["vocab_size"], hidden_size=tc["hidden_size"],
        intermediate_size=tc.get("intermediate_size", 0) or 0,
        num_hidden_layers=tc["num_hidden_layers"], num_attention_heads=heads,
        num_key_value_heads=tc.get("num_key_value_heads", heads),
        head_dim=tc.get("head_dim") or tc["hidden_size"] // heads,
        max_position_embeddings=tc.get("max_position_embeddings", 32768),
        rms_norm_eps=tc.get("rms_norm_eps", 1e-6),
        rope_theta=tc.get("rope_theta") or rope.get("rope_theta", 1e6),
        tie_word_embeddings=bool(tc.get("tie_word_embeddings", root.get("tie_word_embeddings", False))),
    )
    if family != "qwen3_text":
        sec = rope.get("mrope_section")
        if sec is None:
            third = cfg.head_dim // 2 // 3
            sec = [cfg.head_dim // 2 - 2 * third, third, third]
        cfg.mrope_section = list(sec)
    if family == "qwen3_5":
        cfg.offset_norm = True
        cfg.attn_output_gate = True
        cfg.partial_rotary_factor = rope.get("partial_rotary_factor", tc.get("partial_rotary_factor", 0.25))
        cfg.full_attention_interval = tc.get("full_attention_interval", 4)
        cfg.layer_types = list(tc.get("layer_types") or [
            "full_attention" if (i + 1) % cfg.full_attention_interval == 0 else "linear_attention"
            for i in range(cfg.num_hidden_layers)])
        cfg.linear_conv_kernel_dim = tc.get("linear_conv_kernel_dim", 4)
        cfg.linear_key_head_dim = tc.get("linear_key_head_dim", 128)
        cfg.linear_value_head_dim = tc.get("linear_value_head_dim", 128)
        cfg.linear_num_key_heads = tc.get("linear_num_key_heads", 16)
        cfg.linear_num_value_heads = tc.get("linear_num_value_heads", 16)
        if tc.get("num_experts"):
            cfg.num_experts = tc["num_experts"]
            cfg.num_experts_per_tok = tc.get("num_experts_per_tok", 8)
            cfg.moe_intermediate_size = tc.get("moe_intermediate_size", 512)
            cfg.shared_expert_intermediate_size = tc.get("shared_expert_intermediate_size", cfg.moe_intermediate_size)
            cfg.norm_topk_prob = tc.get("norm_topk_prob", True)
    return cfg


def _hybrid_layer_types(n: int, interval: int = 4) -> list[str]:
    return ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(n)]


def _tiny_qwen3() -> ModelConfig:
    return ModelConfig(family="qwen3_text", text=TextConfig(
        vocab_size=151936, hidden_size=256, intermediate_size=768, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e6))


def _qwen3_8b() -> ModelConfig:
    return ModelConfig(family="qwen3_text", text=TextConfig())


def _qwen3_vl_8b() -> ModelConfig:
    return ModelConfig(family="qwen3_vl", text=TextConfig(mrope_section=[24, 20, 20]), vision=VisionConfig())


def _tiny_qwen3_vl() -> ModelConfig:
    return ModelConfig(
        family="qwen3_vl",
        text=TextConfig(vocab_size=152064, hidden_size=128, intermediate_size=256, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=32, mrope_section=[6, 5, 5]),
        vision=VisionConfig(depth=4, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=16,
                            num_position_embeddings=64, out_hidden_size=128, deepstack_visual_indexes=[0, 1, 2]))


def _tiny_qwen3_vl_gpu() -> ModelConfig:
    """Small VLM whose shapes fit the CUDA kernels' tiles (head dims 64 / 72-style padding, dims multiple of 8)."""
    return ModelConfig(
        family="qwen3_vl",
        text=TextConfig(vocab_size=8192, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
                        num_attention_heads=8, num_key_value_heads=4, head_dim=64, mrope_section=[12, 10, 10]),
        vision=VisionConfig(depth=3, hidden_size=288, intermediate_size=576, num_heads=4, patch_size=16,
                            num_position_embeddings=256, out_hidden_size=512, deepstack_visual_indexes=[0, 1, 2]),
        image_token_id=8000, video_token_id=8001, vision_start_token_id=8002, vision_end_token_id=8003)


def _qwen3_5_dense() -> ModelConfig:
    n = 32
    return ModelConfig(family="qwen3_5", vision=None, text=TextConfig(
        vocab_size=248320, hidden_size=4096, intermediate_size=12288, num_hidden_layers=n,
        num_attention_heads=16, num_key_value_heads=4, head_dim=256, rope_theta=1e7,
        mrope_section=[11, 11, 10], partial_rotary_factor=0.25, offset_norm=True, attn_output_gate=True,
        layer_types=_hybrid_layer_types(n), linear_num_key_heads=16, linear_num_value_heads=16,
        linear_key_head_dim=128, linear_value_head_dim=128))


def _qwen3_5_moe() -> ModelConfig:
    n = 40
    return ModelConfig(family="qwen3_5", text=TextConfig(
        vocab_size=248320, hidden_size=2048, intermediate_size=0, num_hidden_layers=n,
        num_attention_heads=16, num_key_value_heads=2, head_dim=256, rope_theta=1e7,
        mrope_section=[11, 11, 10], partial_rotary_factor=0.25, offset_norm=True, attn_output_gate=True,
        layer_types=_hybrid_layer_types(n), linear_num_key_heads=16, linear_num_value_heads=32,
        linear_key_head_dim=128, linear_value_head_dim=128,
        num_experts=256, num_experts_per_tok=8, moe_intermediate_size=512, shared_expert_intermediate_size=512,
        dsa=True),
        vision=VisionConfig(out_hidden_size=2048, deepstack_visual_indexes=[]))


def _tiny_qwen3_5(moe: bool = False) -> ModelConfig:
    n = 4
    t = TextConfig(
        vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=n,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e7,
        mrope_section=[3, 3, 2], partial_rotary_factor=0.25, offset_norm=True, attn_output_gate=True,
        layer_types=_hybrid_layer_types(n), linear_num_key_heads=2, linear_num_value_heads=4,
        linear_key_head_dim=32, linear_value_head_dim=32)
    if moe:
        t.num_experts, t.num_experts_per_tok, t.moe_intermediate_size = 8, 2, 64
        t.shared_expert_intermediate_size, t.intermediate_size = 64, 0
    return ModelConfig(family="qwen3_5", text=t, vision=None)


_PRESETS = {
    "tiny-qwen3": _tiny_qwen3,
    "qwen3-8b": _qwen3_8b,
    "qwen3-vl-8b": _qwen3_vl_8b,
    "tiny-qwen3-vl": _tiny_qwen3_vl,
    "tiny-qwen3-vl-gpu": _tiny_qwen3_vl_gpu,
    "qwen3.5-dense": _qwen3_5_dense,
    "qwen3.5-moe": _qwen3_5_moe,
    "tiny-qwen3.5": _tiny_qwen3_5,
    "tiny-qwen3.5-moe": lambda: _tiny_qwen3_5(True),
}
