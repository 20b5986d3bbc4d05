"""A stock Hugging Face causal LM on one packed row through the registered packed attention must give, document by document,
what the same model gives on the documents one at a time (logits and weight gradients)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _tiny():
    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(0)
    cfg = Qwen3Config(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, max_position_embeddings=64)
    return Qwen3ForCausalLM(cfg)


def test_packed_position_ids_restart_at_every_document():
    from vlm_training_b200.utils.hf_varlen import packed_position_ids

    cu = torch.tensor([0, 3, 4, 9], dtype=torch.int32)
    assert packed_position_ids(cu).tolist() == [[0, 1, 2, 0, 0, 1, 2, 3, 4]]


def test_hf_model_on_a_packed_row_matches_documents_one_by_one():
    from vlm_training_b200.utils import hf_varlen

    model = _tiny()
    docs = [torch.randint(0, 128, (n,)) for n in (5, 7, 1)]
    losses = [model(input_ids=d[None]).logits.float().pow(2).mean() * d.numel() for d in docs]
    sum(losses).backward()
    want_logits = torch.cat([model(input_ids=d[None]).logits[0] for d in docs]).detach()
    want_grad = model.model.layers[0].self_attn.q_proj.weight.grad.clone()
    model.zero_grad()

    hf_varlen.enable(model)
    assert model.config._attn_implementation == hf_varlen.NAME
    cu = torch.tensor([0, 5, 12, 13], dtype=torch.int32)
    out = model(input_ids=torch.cat(docs)[None], position_ids=hf_varlen.packed_position_ids(cu), cu_seqlens=cu).logits[0]
    assert torch.allclose(out, want_logits, atol=1e-5, rtol=1e-5)
    # the same loss as above: every document's mean of squares times its length = the packed row's sum / vocab
    (out.float().pow(2).sum() / out.shape[-1]).backward()
    got_grad = model.model.layers[0].self_attn.q_proj.weight.grad
    assert torch.allclose(got_grad, want_grad, atol=1e-5, rtol=1e-4)


def test_packed_attention_demands_cu_seqlens():
    from vlm_training_b200.utils import hf_varlen

    model = hf_varlen.enable(_tiny())
    with pytest.raises(ValueError, match="cu_seqlens"):
        model(input_ids=torch.randint(0, 128, (1, 6)))
