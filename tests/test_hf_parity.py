"""Logit / loss parity of the native models against HF ``transformers`` modules
built from the same config with the same random weights (fp32, CPU).

Mirrors the reference's parity suite (reference: models/tests/test_qwen3_parity.py:62-77,
test_qwen3_vl_full_parity.py:77-98, test_qwen3_5_exhaustive.py:203-263) without
needing a snapshot: weights are copied from the HF module through the native
``load_state_dict`` (which also exercises the fused-parameter key mapping).
"""
import pytest
import torch

from vlm_training_b200.models import ModelConfig, build_model

torch.manual_seed(0)


def _hf_qwen3(cfg):
    from transformers import Qwen3Config, Qwen3ForCausalLM

    t = cfg.text
    hc = Qwen3Config(vocab_size=t.vocab_size, hidden_size=t.hidden_size, intermediate_size=t.intermediate_size,
                     num_hidden_layers=t.num_hidden_layers, num_attention_heads=t.num_attention_heads,
                     num_key_value_heads=t.num_key_value_heads, head_dim=t.head_dim, rms_norm_eps=t.rms_norm_eps,
                     rope_theta=t.rope_theta, tie_word_embeddings=False, attention_bias=False,
                     max_position_embeddings=4096)
    hc._attn_implementation = "eager"
    return Qwen3ForCausalLM(hc).eval()


def test_qwen3_text_logits_match_hf():
    cfg = ModelConfig.preset("tiny-qwen3", vocab_size=512)
    hf = _hf_qwen3(cfg)
    ours = build_model(cfg, init=False)
    missing = ours.load_state_dict(hf.state_dict(), strict=True)
    ids = torch.randint(0, 512, (1, 48))
    with torch.no_grad():
        ref = hf(ids).logits
        got = ours(ids)
    assert torch.equal(ref.argmax(-1), got.argmax(-1))
    torch.testing.assert_close(got, ref, atol=1e-3, rtol=1e-3)


def test_qwen3_text_loss_and_packing():
    cfg = ModelConfig.preset("tiny-qwen3", vocab_size=512)
    hf = _hf_qwen3(cfg)
    ours = build_model(cfg, init=False)
    ours.load_state_dict(hf.state_dict())
    a, b = torch.randint(0, 512, (1, 40)), torch.randint(0, 512, (1, 25))
    with torch.no_grad():
        la = hf(a, labels=a).loss
        got = ours(a, labels=a).loss
        assert abs(la.item() - got.item()) < 1e-3
        # packed row == solo rows (varlen self-consistency)
        packed = torch.cat((a, b), 1)
        cu = torch.tensor([0, 40, 65])
        lp = ours(packed, attention_mask=cu)
        torch.testing.assert_close(lp[:, :40], ours(a), atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(lp[:, 40:], ours(b), atol=1e-4, rtol=1e-4)


def _hf_qwen3_vl(cfg):
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    t, v = cfg.text, cfg.vision
    hc = Qwen3VLConfig(
        text_config=dict(vocab_size=t.vocab_size, hidden_size=t.hidden_size, intermediate_size=t.intermediate_size,
                         num_hidden_layers=t.num_hidden_layers, num_attention_heads=t.num_attention_heads,
                         num_key_value_heads=t.num_key_value_heads, head_dim=t.head_dim, rms_norm_eps=t.rms_norm_eps,
                         rope_theta=t.rope_theta, max_position_embeddings=4096,
                         rope_scaling={"rope_type": "default", "mrope_section": t.mrope_section, "mrope_interleaved": True}),
        vision_config=dict(depth=v.depth, hidden_size=v.hidden_size, intermediate_size=v.intermediate_size,
                           num_heads=v.num_heads, in_channels=3, patch_size=v.patch_size,
                           temporal_patch_size=v.temporal_patch_size, spatial_merge_size=v.spatial_merge_size,
                           num_position_embeddings=v.num_position_embeddings, out_hidden_size=v.out_hidden_size,
                           hidden_act=v.hidden_act, deepstack_visual_indexes=v.deepstack_visual_indexes),
        image_token_id=cfg.image_token_id, video_token_id=cfg.video_token_id,
        vision_start_token_id=cfg.vision_start_token_id, vision_end_token_id=cfg.vision_end_token_id,
        tie_word_embeddings=False)
    hc._attn_implementation = "eager"
    hc.text_config._attn_implementation = "eager"
    hc.vision_config._attn_implementation = "eager"
    return Qwen3VLForConditionalGeneration(hc).eval()


def _vl_row(cfg, grids, n_text=7):
    ids = []
    for (t, h, w) in grids:
        ids += torch.randint(0, 1000, (n_text,)).tolist()
        ids += [cfg.vision_start_token_id] + [cfg.image_token_id] * (t * h * w // 4) + [cfg.vision_end_token_id]
    ids += torch.randint(0, 1000, (n_text,)).tolist()
    n_patches = sum(t * h * w for t, h, w in grids)
    pixels = torch.randn(n_patches, cfg.vision.patch_dim)
    return torch.tensor([ids]), pixels, torch.tensor(grids)


def test_qwen3_vl_multimodal_logits_match_hf():
    cfg = ModelConfig.preset("tiny-qwen3-vl")
    hf = _hf_qwen3_vl(cfg)
    ours = build_model(cfg, init=False)
    ours.load_state_dict(hf.state_dict(), strict=True)
    ids, pixels, grids = _vl_row(cfg, [(1, 4, 4), (1, 2, 6)])
    with torch.no_grad():
        mm = (ids == cfg.image_token_id).int()
        ref = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grids, mm_token_type_ids=mm).logits
        got = ours(ids, pixel_values=pixels, image_grid_thw=grids)
    assert torch.equal(ref.argmax(-1), got.argmax(-1))
    torch.testing.assert_close(got, ref, atol=2e-3, rtol=2e-3)


def test_qwen3_vl_vision_tower_matches_hf():
    cfg = ModelConfig.preset("tiny-qwen3-vl")
    hf = _hf_qwen3_vl(cfg)
    ours = build_model(cfg, init=False)
    ours.load_state_dict(hf.state_dict())
    grids = torch.tensor([[1, 4, 4], [1, 2, 6]])
    pixels = torch.randn(28, cfg.vision.patch_dim)
    with torch.no_grad():
        out = hf.model.visual(pixels, grid_thw=grids)
        merged, deep = ours.visual(pixels, grids)
    ref_merged = out.pooler_output if hasattr(out, "pooler_output") else out[0]
    ref_deep = out.deepstack_features if hasattr(out, "deepstack_features") else out[1]
    torch.testing.assert_close(merged, ref_merged, atol=1e-3, rtol=1e-3)
    for a, b in zip(deep, ref_deep):
        torch.testing.assert_close(a, b, atol=1e-3, rtol=1e-3)


def _hf_qwen3_5(cfg, moe=False):
    t = cfg.text
    common = dict(vocab_size=t.vocab_size, hidden_size=t.hidden_size, num_hidden_layers=t.num_hidden_layers,
                  num_attention_heads=t.num_attention_heads, num_key_value_heads=t.num_key_value_heads,
                  head_dim=t.head_dim, rms_norm_eps=t.rms_norm_eps, max_position_embeddings=4096,
                  layer_types=t.layer_types, full_attention_interval=t.full_attention_interval,
                  linear_conv_kernel_dim=t.linear_conv_kernel_dim, linear_key_head_dim=t.linear_key_head_dim,
                  linear_value_head_dim=t.linear_value_head_dim, linear_num_key_heads=t.linear_num_key_heads,
                  linear_num_value_heads=t.linear_num_value_heads, tie_word_embeddings=False,
                  rope_parameters={"rope_type": "default", "rope_theta": t.rope_theta,
                                   "partial_rotary_factor": t.partial_rotary_factor,
                                   "mrope_section": t.mrope_section, "mrope_interleaved": True})
    if moe:
        from transformers.models.qwen3_5_moe import Qwen3_5MoeTextConfig
        from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM

        hc = Qwen3_5MoeTextConfig(**common, num_experts=t.num_experts, num_experts_per_tok=t.num_experts_per_tok,
                                  moe_intermediate_size=t.moe_intermediate_size,
                                  shared_expert_intermediate_size=t.shared_expert_intermediate_size)
        hc._attn_implementation = "eager"
        return Qwen3_5MoeForCausalLM(hc).eval()
    from transformers.models.qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM

    hc = Qwen3_5TextConfig(**common, intermediate_size=t.intermediate_size)
    hc._attn_implementation = "eager"
    return Qwen3_5ForCausalLM(hc).eval()


def _load_text_only(ours, hf):
    # HF text-only CausalLM uses "model.*"; the native VLM layout nests it under model.language_model.*
    sd = {}
    for k, v in hf.state_dict().items():
        sd[k.replace("model.", "model.language_model.", 1) if k.startswith("model.") else k] = v
    return ours.load_state_dict(sd, strict=True)


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_5_text_logits_match_hf(moe):
    cfg = ModelConfig.preset("tiny-qwen3.5-moe" if moe else "tiny-qwen3.5")
    hf = _hf_qwen3_5(cfg, moe)
    with torch.no_grad():  # make the comparison non-trivial: HF zero-inits the router and offset norms
        for n, p in hf.named_parameters():
            if "norm" in n or n.endswith("gate.weight"):
                p.add_(torch.randn_like(p) * 0.1)
    ours = build_model(cfg, init=False)
    _load_text_only(ours, hf)
    ids = torch.randint(0, cfg.text.vocab_size, (1, 150))  # spans several 64-token GDN chunks
    with torch.no_grad():
        ref = hf(ids).logits
        got = ours(ids)
    assert (ref.argmax(-1) == got.argmax(-1)).float().mean() > 0.99
    torch.testing.assert_close(got, ref, atol=2e-3, rtol=2e-3)


def test_qwen3_5_packed_equals_solo():
    """Recurrent state, conv taps and attention must not leak across documents
    (reference: models/tests/test_qwen3_5_loss_parity.py:96-129)."""
    cfg = ModelConfig.preset("tiny-qwen3.5")
    ours = build_model(cfg, seed=1)
    a, b, c = (torch.randint(0, 1024, (1, n)) for n in (70, 33, 129))
    packed = torch.cat((a, b, c), 1)
    cu = torch.tensor([0, 70, 103, 232])
    with torch.no_grad():
        lp = ours(packed, attention_mask=cu)
        for s, e, solo in ((0, 70, a), (70, 103, b), (103, 232, c)):
            torch.testing.assert_close(lp[:, s:e], ours(solo), atol=2e-4, rtol=2e-4)
