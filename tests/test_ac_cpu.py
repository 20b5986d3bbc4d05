"""Activation checkpointing policies give the same loss and gradients as no checkpointing (CPU, fp32)."""
import pytest
import torch


def _run(mode: str, preset: str):
    from vlm_training_b200.models import ModelConfig, build_model
    from vlm_training_b200.parallel.ac import apply_ac

    torch.manual_seed(0)
    cfg = ModelConfig.preset(preset)
    cfg.text.vocab_size = 512
    model = build_model(cfg, dtype=torch.float32, device="cpu")
    apply_ac(model, mode)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (96,), generator=g)
    cu = torch.tensor([0, 40, 96], dtype=torch.int32)
    out = model(ids, attention_mask=cu, labels=ids)
    out.loss.backward()
    return out.loss.detach(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("preset", ["tiny-qwen3", "tiny-qwen3.5"])
@pytest.mark.parametrize("mode", ["full", "sac"])
def test_checkpointed_backward_matches_plain(mode, preset):
    loss0, g0 = _run("off", preset)
    loss1, g1 = _run(mode, preset)
    assert torch.allclose(loss0, loss1, rtol=0, atol=1e-6)
    assert g0.keys() == g1.keys()
    for n in g0:
        assert torch.allclose(g0[n], g1[n], rtol=1e-5, atol=1e-6), n


def test_sac_recomputes_only_the_mlp_half(monkeypatch):
    """Under ``sac`` the mixer half runs once per layer and step, the MLP half twice (forward + recomputation)."""
    from vlm_training_b200.models import ModelConfig, build_model
    from vlm_training_b200.models.layers import DecoderLayer
    from vlm_training_b200.parallel.ac import apply_ac

    calls = {"mixer": 0, "mlp": 0}
    mixer, mlp = DecoderLayer.mixer_half, DecoderLayer.mlp_half
    monkeypatch.setattr(DecoderLayer, "mixer_half", lambda self, x, ctx: (calls.__setitem__("mixer", calls["mixer"] + 1), mixer(self, x, ctx))[1])
    monkeypatch.setattr(DecoderLayer, "mlp_half", lambda self, h, x: (calls.__setitem__("mlp", calls["mlp"] + 1), mlp(self, h, x))[1])
    cfg = ModelConfig.preset("tiny-qwen3")
    cfg.text.vocab_size = 512
    model = build_model(cfg, dtype=torch.float32, device="cpu")
    apply_ac(model, "sac")
    ids = torch.randint(0, 512, (64,))
    model(ids, labels=ids).loss.backward()
    n = cfg.text.num_hidden_layers
    assert calls == {"mixer": n, "mlp": 2 * n}


def test_unknown_block_rejects_sac():
    from vlm_training_b200.parallel.ac import checkpoint_layer

    with pytest.raises(ValueError):
        checkpoint_layer(torch.nn.Identity(), torch.zeros(1), None, "sac")
