from .config import ModelConfig, TextConfig, VisionConfig
from .causal_lm import (BatchPlan, CausalLMOutput, MODEL_CLASSES, Qwen3ForCausalLM, Qwen3VLForCausalLM,
                        Qwen3_5ForCausalLM, build_model)

__all__ = ["ModelConfig", "TextConfig", "VisionConfig", "BatchPlan", "CausalLMOutput", "MODEL_CLASSES",
           "Qwen3ForCausalLM", "Qwen3VLForCausalLM", "Qwen3_5ForCausalLM", "build_model"]
