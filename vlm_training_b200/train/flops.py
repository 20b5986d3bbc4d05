"""Model FLOPs per token (Megatron-style accounting) and MFU.

Conventions follow the reference estimator (reference: train/flops_estimation.py:19-200):
every GEMM counts 2 FLOPs per multiply-add and x3 for forward + dgrad + wgrad; causal
attention counts half of the score matrix; the Gated-DeltaNet recurrence is approximated
by ``n_v * d_v^2 * 4`` per token; the ViT is charged per LLM token at the LLM sequence
length.  Added here: text-only Qwen3 (the reference raises for it) and MoE layers
(router + top-k routed experts + shared expert).
"""
from __future__ import annotations

from ..models.config import ModelConfig, TextConfig, VisionConfig

FWD_BWD = 3
FMA = 2


def _mlp(hidden: int, inter: int, swiglu: bool) -> float:
    return inter * (3 if swiglu else 2) * hidden * FWD_BWD * FMA


def _attention(head_dim, n_heads, n_kv, hidden, seq_len, gate=False, causal=True) -> float:
    q, kv = head_dim * n_heads, head_dim * n_kv
    proj = hidden * (q + 2 * kv + (q if gate else 0))
    core = q * seq_len / (2 if causal else 1) * 2
    return FWD_BWD * FMA * (proj + core + q * hidden)


def _gdn(t: TextConfig) -> float:
    qk, v = t.linear_key_head_dim * t.linear_num_key_heads, t.linear_value_head_dim * t.linear_num_value_heads
    return FWD_BWD * FMA * (t.hidden_size * (2 * qk + 2 * v + 2 * t.linear_num_value_heads)
                            + t.linear_conv_kernel_dim * (2 * qk + v)
                            + t.linear_num_value_heads * t.linear_value_head_dim ** 2 * 4
                            + t.hidden_size * v)


def _moe(t: TextConfig) -> float:
    routed = t.num_experts_per_tok * _mlp(t.hidden_size, t.moe_intermediate_size, True)
    shared = _mlp(t.hidden_size, t.shared_expert_intermediate_size, True)
    router = FWD_BWD * FMA * t.hidden_size * (t.num_experts + 1)
    return routed + shared + router


def vision_flops_per_token(v: VisionConfig, seq_len: int) -> float:
    att = _attention(v.head_dim, v.num_heads, v.num_heads, v.hidden_size, seq_len, causal=True)
    return v.depth * (att + _mlp(v.hidden_size, v.intermediate_size, False))


def text_flops_per_token(t: TextConfig, seq_len: int) -> dict:
    n = t.num_hidden_layers
    n_full = sum(1 for i in range(n) if t.layer_type(i) == "full_attention")
    n_lin = n - n_full
    att = _attention(t.head_dim, t.num_attention_heads, t.num_key_value_heads, t.hidden_size, seq_len, gate=t.attn_output_gate)
    mlp = _moe(t) if t.num_experts > 0 else _mlp(t.hidden_size, t.intermediate_size, True)
    out = {"attention": att * n_full, "linear_attention": (_gdn(t) * n_lin) if n_lin else 0.0, "mlp": mlp * n,
           "logits": FWD_BWD * FMA * t.hidden_size * t.vocab_size}
    out["total"] = sum(out.values())
    return out


def flops_per_token(cfg: ModelConfig, seq_len: int) -> float:
    total = text_flops_per_token(cfg.text, seq_len)["total"]
    if cfg.vision is not None:
        total += vision_flops_per_token(cfg.vision, seq_len)
    return total


def get_dense_model_nparams_and_flops(cfg: ModelConfig, model, seq_len: int) -> tuple[int, int]:
    """(parameter count, FLOPs per token) — same call shape as the reference helper
    (reference: train/flops_estimation.py:7-17)."""
    return int(sum(p.numel() for p in model.parameters())), int(flops_per_token(cfg, seq_len))


def peak_flops(device_name: str | None = None) -> float:
    """bf16 dense peak used as the MFU denominator.  The reference hard-codes the H100 value
    (989.4 TFLOP/s, reference: train/train_qwen.py:142-144); here it is read from the measured
    peaks file when present, else the B200 nominal 2.25 PFLOP/s."""
    import json
    import os

    for path in (os.environ.get("VLMT_MEASURED_PEAKS", ""), "MEASURED_PEAKS.json"):
        if path and os.path.exists(path):
            try:
                with open(path) as fh:
                    return float(json.load(fh)["bf16_tflops_sustained"]) * 1e12
            except Exception:
                pass
    return 2.25e15
