"""Config loader / CLI overrides, schedulers, accumulation pattern, FLOPs model, optimizer groups, packing."""
import math
import random

import pytest
import torch

from vlm_training_b200.config import Config, ConfigManager, ModelType
from vlm_training_b200.data.packing import assistant_label_mask, collate_row, select_bins
from vlm_training_b200.models import ModelConfig, build_model
from vlm_training_b200.train import flops
from vlm_training_b200.train.optimizer import build_param_groups, group_of
from vlm_training_b200.train.schedulers import accumulation_pattern, cosine_multiplier, wsd_multiplier


def test_toml_then_cli_precedence(tmp_path):
    f = tmp_path / "c.toml"
    f.write_text('[model]\nmodel_name = "Qwen3-VL-8B"\n[training]\ntp_size = 2\nlr_llm = 1e-5\n[data]\nseq_len = 4096\n')
    cfg = ConfigManager(Config).parse_args(["--config", str(f), "--training.tp_size", "4", "--data.seq_len=8192",
                                            "--training.sequence_parallel"])
    assert cfg.model.model_name == "Qwen3-VL-8B" and cfg.training.tp_size == 4 and cfg.training.lr_llm == 1e-5
    assert cfg.data.seq_len == 8192 and cfg.training.sequence_parallel is True and cfg.config == str(f)
    assert Config().training.tp_size == 1  # defaults untouched


def test_unknown_keys_are_errors(tmp_path):
    f = tmp_path / "c.toml"
    f.write_text("[training]\nrandom_init_mlp = true\n")  # a key some of the reference's shipped TOMLs carry
    with pytest.raises(ValueError, match="random_init_mlp"):
        ConfigManager(Config).parse_args(["--config", str(f)])
    with pytest.raises(ValueError):
        ConfigManager(Config).parse_args(["--training.nope", "1"])


def test_every_shipped_config_loads():
    import glob
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = glob.glob(os.path.join(root, "configs", "*.toml"))
    assert files
    for f in files:
        ConfigManager(Config).parse_args(["--config", f])


def test_model_type_from_name():
    assert ModelType.from_name("Qwen3.5-9B") is ModelType.QWEN3_5
    assert ModelType.from_name("Qwen3-VL-8B-Instruct") is ModelType.QWEN3_VL
    assert ModelType.from_name("Qwen3-1.7B") is ModelType.QWEN3_TEXT


def test_schedulers_match_their_formulas():
    f = wsd_multiplier(total_steps=100, warmup_steps=10, decay_ratio=0.2)
    assert f(0) == 0 and f(5) == 0.5 and f(10) == 1 and f(79) == 1
    assert f(80) == pytest.approx(1.0) and f(90) == pytest.approx(0.5) and f(100) == pytest.approx(0.0, abs=1e-9)
    g = cosine_multiplier(total_steps=100, warmup_steps=10, min_lr_ratio=0.1)
    assert g(5) == 0.5 and g(10) == pytest.approx(1.0) and g(100) == pytest.approx(0.1)
    assert g(55) == pytest.approx(0.1 + 0.9 * 0.5)


@pytest.mark.parametrize("m,expect", [(1.0, [1]), (1.5, [1, 2]), (2.0, [2]), (1.25, [1, 1, 1, 2])])
def test_accumulation_pattern(m, expect):
    pat = accumulation_pattern(m)
    assert pat == expect and sum(pat) / len(pat) == pytest.approx(m)


def test_flops_model_matches_hand_count():
    cfg = ModelConfig.preset("qwen3-8b")
    t = cfg.text
    S = 8192
    per_layer = 6 * (t.hidden_size * (t.num_attention_heads + 2 * t.num_key_value_heads) * t.head_dim
                     + t.num_attention_heads * t.head_dim * S / 2 * 2 + t.num_attention_heads * t.head_dim * t.hidden_size
                     + 3 * t.intermediate_size * t.hidden_size)
    total = per_layer * t.num_hidden_layers + 6 * t.hidden_size * t.vocab_size
    assert flops.flops_per_token(cfg, S) == pytest.approx(total)
    moe = ModelConfig.preset("qwen3.5-moe")
    assert flops.text_flops_per_token(moe.text, 4096)["linear_attention"] > 0
    assert flops.flops_per_token(moe, 4096) > 0


def test_three_learning_rate_groups():
    assert group_of("model.visual.merger.linear_fc1.weight") == "mlp"
    assert group_of("model.visual.deepstack_merger_list.0.norm.weight") == "mlp"
    assert group_of("model.visual.blocks.3.attn.qkv.weight") == "vit"
    assert group_of("model.language_model.layers.0.mlp.gate_up.weight") == "llm"
    model = build_model(ModelConfig.preset("tiny-qwen3-vl"), init=False)
    groups = build_param_groups(model, 2e-6, 1e-5, 1e-6, 0.01)
    lrs = {g.name: g.lr for g in groups}
    assert lrs["llm"] == 2e-6 and lrs["mlp"] == 1e-5 and lrs["vit"] == 1e-6
    assert all(g.weight_decay == 0 for g in groups if g.name.endswith("_nodecay"))
    n = sum(len(g.params) for g in groups)
    assert n == sum(1 for p in model.parameters() if p.requires_grad)


def test_packing_bins_and_collate():
    lens = [900, 100, 500, 450, 60, 2000]
    bins = select_bins(lens, 1024, random.Random(0))
    assert sorted(i for b in bins for i in b) == list(range(len(lens)))
    for b in bins:
        assert sum(lens[i] for i in b) <= 1024 or len(b) == 1  # an over-long sample sits alone
    samples = [{"input_ids": torch.arange(n), "labels": torch.arange(n)} for n in (5, 3)]
    row = collate_row(samples, 12, pad_token_id=99)
    assert row["cu_seqlens"].tolist() == [0, 5, 8, 12]  # the pad tail is its own segment
    assert row["input_ids"][8:].tolist() == [99] * 4 and row["labels"][8:].tolist() == [-100] * 4


def test_assistant_label_mask_keeps_answer_and_eos():
    A, EOS = 7, 2
    ids = [1, A, 9, 5, 6, EOS, 3, A, 9, 8, EOS, 4]
    lab = assistant_label_mask(ids, A, EOS).tolist()
    assert lab == [-100, -100, -100, 5, 6, EOS, 3, -100, -100, 8, EOS, 4]


def test_synthetic_rows_have_the_named_shape():
    from vlm_training_b200.data.synthetic import SyntheticDataset, SyntheticSpec

    cfg = ModelConfig.preset("tiny-qwen3-vl")
    b = next(SyntheticDataset(SyntheticSpec(kind="vlm", seq_len=2048, vocab_size=cfg.text.vocab_size), cfg))
    assert b["input_ids"].numel() == 2048 and b["cu_seqlens"][0] == 0 and b["cu_seqlens"][-1] == 2048
    g = b["image_grid_thw"]
    assert ((g[:, 1] * 16 >= 224) & (g[:, 1] * 16 <= 1024) & (g[:, 1] % 2 == 0)).all()
    assert int((b["input_ids"] == cfg.image_token_id).sum()) == int((g[:, 0] * (g[:, 1] // 2) * (g[:, 2] // 2)).sum())
    assert b["pixel_values"].shape == (int((g[:, 0] * g[:, 1] * g[:, 2]).sum()), 1536)
    assert (b["labels"][b["cu_seqlens"][:-1].long()] == -100).all()  # no prediction across document boundaries
    t = next(SyntheticDataset(SyntheticSpec(kind="text-loguniform", seq_len=4096, doc_len_min=128, doc_len_max=4096), cfg))
    assert t["input_ids"].numel() == 4096


def test_dcp_to_hf_conversion_roundtrip(tmp_path):
    """Trainer checkpoint → converter → safetensors snapshot → from_pretrained gives the trained weights back."""
    from vlm_training_b200.models import config as mc
    from vlm_training_b200.models.causal_lm import Qwen3ForCausalLM
    from vlm_training_b200.train.trainer import Trainer
    from vlm_training_b200.utils.convert import convert

    orig = mc._PRESETS["tiny-qwen3"]

    def small():
        c = orig()
        c.text.vocab_size = 512
        return c

    mc._PRESETS["tiny-qwen3"] = small
    try:
        cfg = Config()
        cfg.model.model_name, cfg.model.preset = "Qwen3-tiny", "tiny-qwen3"
        t = cfg.training
        t.output_dir, t.bfloat16, t.device, t.total_steps, t.save_steps, t.warmup_steps = str(tmp_path / "ck"), False, "cpu", 2, 2, 0
        cfg.data.synthetic, cfg.data.seq_len, cfg.data.doc_len_min, cfg.data.doc_len_max = "text-uniform", 128, 16, 64
        tr = Trainer(cfg)
        tr.train()
        want = {k: v.clone() for k, v in tr.model.state_dict().items()}
        out = convert(t.output_dir, "tiny-qwen3", str(tmp_path / "hf"), dtype=torch.float32)
        assert out and out[0].endswith("step-2")
        import json

        json.dump({"vocab_size": 512, "hidden_size": 256, "intermediate_size": 768, "num_hidden_layers": 2, "num_attention_heads": 4,
                   "num_key_value_heads": 2, "head_dim": 64, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 4096,
                   "tie_word_embeddings": False}, open(out[0] + "/config.json", "w"))
        model, _ = Qwen3ForCausalLM.from_pretrained(out[0], dtype=torch.float32)
        for k, v in model.state_dict().items():
            torch.testing.assert_close(v, want[k])
    finally:
        mc._PRESETS["tiny-qwen3"] = orig


def test_energon_items_are_normalised_cooked_and_sharded(monkeypatch):
    """The energon path end to end on our side, with a stand-in for the (not installed) package: items arrive as batches
    of one with raw bytes, leave as cooked ``{"image", "messages"}`` samples; rank and worker count reach the loader."""
    import io
    import json as _json
    import sys
    import types

    from PIL import Image

    from vlm_training_b200.config import Config
    from vlm_training_b200.data import task_encoders as te

    buf = io.BytesIO()
    Image.new("RGB", (8, 8), (255, 0, 0)).save(buf, format="PNG")
    crude = [[{"__key__": f"s{i}", "jpg": buf.getvalue(),
               "json": _json.dumps({"conversations": [{"from": "human", "value": "<image>\nwhat?"}, {"from": "gpt", "value": f"red {i}"}]}).encode()}]
             for i in range(3)]
    seen = {}
    fake = types.ModuleType("megatron.energon")

    class WorkerConfig:
        def __init__(self, rank, world_size, num_workers):
            seen.update(rank=rank, world=world_size, workers=num_workers)

    fake.WorkerConfig = WorkerConfig
    fake.get_train_dataset = lambda path, **kw: ("dataset", path, kw)
    fake.get_loader = lambda ds: iter(crude)
    monkeypatch.setitem(sys.modules, "megatron", types.ModuleType("megatron"))
    monkeypatch.setitem(sys.modules, "megatron.energon", fake)
    d = Config().data
    d.num_workers = 3
    out = list(te._energon_samples("/data/x", d, rank=1, world=4))
    assert seen == {"rank": 1, "world": 4, "workers": 3}
    assert len(out) == 3 and all(set(o) >= {"image", "messages"} for o in out)
    assert out[0]["image"].size == (8, 8)
    assert [m["role"] for m in out[2]["messages"]] == ["user", "assistant"]
    assert out[2]["messages"][0]["content"][0] == {"type": "image"}
    assert out[2]["messages"][1]["content"][0]["text"] == "red 2"
    # captions: the cooker follows the sample's fields
    assert te.pick_cooker({"jpg": None, "txt": "a cat"}) is te.cookers.cook_llava_imagenet
    import pytest as _pytest

    with _pytest.raises(KeyError):
        te.pick_cooker({"jpg": None})
