"""Every model family end to end on the GPU (bf16, CUDA kernels) against the same weights on the CPU (fp32, plain
PyTorch reference ops): loss and a few gradients must agree within bf16 tolerances."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from vlm_training_b200.data.synthetic import SyntheticDataset, SyntheticSpec
from vlm_training_b200.models import BatchPlan, ModelConfig, build_model


def _batch(cfg, kind, seq_len):
    spec = SyntheticSpec(kind=kind, seq_len=seq_len, vocab_size=cfg.text.vocab_size, doc_len_min=32, doc_len_max=256,
                         side_min=64, side_max=160, seed=3)
    return next(SyntheticDataset(spec, cfg))


def _run(model, cfg, batch, device):
    ids = batch["input_ids"].to(device)
    cu = batch["cu_seqlens"]
    grids = batch["image_grid_thw"].tolist() if "image_grid_thw" in batch else None
    plan = BatchPlan.build(cfg, batch["input_ids"], cu, grids, device)
    kw = {}
    if grids is not None:
        kw = dict(pixel_values=batch["pixel_values"].to(device=device, dtype=next(model.parameters()).dtype),
                  image_grid_thw=batch["image_grid_thw"])
    out = model(ids, attention_mask=cu.to(device), labels=batch["labels"].to(device), batch_plan=plan, **kw)
    out.loss.backward()
    return out.loss.detach().float().cpu()


CASES = [
    ("tiny-qwen3", "text-uniform", 512, {}),
    ("tiny-qwen3-vl-gpu", "vlm", 1024, {}),
    ("tiny-qwen3.5", "text-uniform", 512, {}),
    ("tiny-qwen3.5-moe", "text-uniform", 512, {}),
    ("tiny-qwen3.5", "text-uniform", 512, {"dsa": True}),
]


@pytest.mark.parametrize("preset,kind,seq_len,over", CASES)
def test_family_gpu_matches_cpu_reference(preset, kind, seq_len, over):
    from vlm_training_b200.ops import cuda as cu

    torch.manual_seed(0)
    cfg = ModelConfig.preset(preset)
    cfg.text.vocab_size = min(cfg.text.vocab_size, 8192)
    for k, v in over.items():
        setattr(cfg.text, k, v)
    if over.get("dsa"):
        cfg.text.dsa_topk = 64
    ref_model = build_model(cfg, dtype=torch.float32, device="cpu")
    from vlm_training_b200.models.init import init_normal_

    init_normal_(ref_model, seed=1)
    gpu_model = copy.deepcopy(ref_model).to(device="cuda", dtype=torch.bfloat16)
    ref_model = copy.deepcopy(gpu_model).to(device="cpu", dtype=torch.float32)   # same (bf16-rounded) weights
    batch = _batch(cfg, kind, seq_len)
    loss_gpu = _run(gpu_model, cfg, batch, "cuda")
    cu.check_status()
    loss_cpu = _run(ref_model, cfg, batch, "cpu")
    assert torch.isfinite(loss_gpu)
    assert abs(float(loss_gpu) - float(loss_cpu)) < 3e-2 * max(1.0, abs(float(loss_cpu))), (float(loss_gpu), float(loss_cpu))
    # gradients: every parameter gets one, and the big ones agree in direction and size
    checked = 0
    for (n, pg), (_, pc) in zip(gpu_model.named_parameters(), ref_model.named_parameters()):
        # same parameters take part in the loss on both paths (the DSA indexer only selects keys: no gradient on either)
        assert (pg.grad is None) == (pc.grad is None), n
        if pg.grad is None:
            continue
        g, c = pg.grad.float().cpu().flatten(), pc.grad.float().flatten()
        assert torch.isfinite(g).all(), n
        if c.numel() >= 4096 and float(c.norm()) > 1e-6:
            cos = float(torch.dot(g, c) / (g.norm() * c.norm() + 1e-12))
            assert cos > 0.97, (n, cos)
            assert 0.8 < float(g.norm() / c.norm()) < 1.25, (n, float(g.norm() / c.norm()))
            checked += 1
    assert checked > 0
