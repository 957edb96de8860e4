"""Hugging Face GPT-2 / BERT models with their FFN blocks converted to MoE layers (CPU, tiny random models)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from ccfuser_b200 import MoELayer  # noqa: E402
from ccfuser_b200.models.hf import aux_loss, convert_bert, convert_gpt2  # noqa: E402
from ccfuser_b200.parallel.ddp import expert_param_names  # noqa: E402


def test_gpt2_blocks_become_moe_and_train():
    from transformers import GPT2Config, GPT2LMHeadModel
    torch.manual_seed(0)
    model = GPT2LMHeadModel(GPT2Config(n_layer=4, n_head=2, n_embd=32, vocab_size=128, n_positions=32,
                                       resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0))
    layers = convert_gpt2(model, num_experts=4, top_k=2, every=2, max_tokens=64)
    assert len(layers) == 2 and all(isinstance(l, MoELayer) for l in layers)
    assert isinstance(model.transformer.h[1].mlp.moe, MoELayer) and isinstance(model.transformer.h[3].mlp.moe, MoELayer)
    assert not hasattr(model.transformer.h[0].mlp, "moe")
    sd = model.state_dict()
    assert sd["transformer.h.1.mlp.moe.experts.htoh4.weight"].shape == (4, 128, 32)
    assert sd["transformer.h.1.mlp.moe.gate.gate.weight"].shape == (4, 32)
    names = expert_param_names(model)
    assert len(names) == 2 * 4 and all(".experts." in n for n in names)
    ids = torch.randint(0, 128, (2, 32))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]
    assert layers[0].experts.htoh4.weight.grad.abs().sum() > 0 and layers[0].gate.gate.weight.grad.abs().sum() > 0


def test_bert_qa_layers_become_moe():
    from transformers import BertConfig, BertForQuestionAnswering
    torch.manual_seed(0)
    model = BertForQuestionAnswering(BertConfig(num_hidden_layers=4, num_attention_heads=2, hidden_size=32,
                                                intermediate_size=64, vocab_size=128, max_position_embeddings=32,
                                                hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0))
    layers = convert_bert(model, num_experts=4, top_k=2, layers=(1, 3), max_tokens=64)
    for l in layers:
        l.gate.aux_loss_coef = 0.01
    assert len(layers) == 2
    assert isinstance(model.bert.encoder.layer[1].intermediate.moe, MoELayer)
    assert sum(p.numel() for p in model.bert.encoder.layer[1].output.dense.parameters()) == 0
    ids = torch.randint(0, 128, (2, 32))
    out = model(input_ids=ids, start_positions=torch.tensor([1, 2]), end_positions=torch.tensor([3, 4]))
    assert out.start_logits.shape == (2, 32)
    extra = aux_loss(layers)
    assert extra is not None and float(extra) > 0
    (out.loss + extra).backward()
    assert layers[1].experts.h4toh.weight.grad.abs().sum() > 0
    assert model.bert.encoder.layer[3].output.LayerNorm.weight.grad is not None


def test_hf_example_trainer_runs_both_models_on_cpu():
    from ccfuser_b200.examples import hf_train
    common = ["--steps", "2", "--warmup", "0", "--layers", "4", "--heads", "2", "--hidden", "32", "--vocab", "128", "--batch", "2",
              "--seq", "16", "--experts-per-gpu", "4", "--dtype", "fp32"]
    for model, n_moe in (("gpt2", 4), ("bert", 1)):
        for variant in ("dense", "nccl"):
            out = hf_train.main(["--model", model, "--variant", variant] + common)
            assert out["moe_layers"] == (0 if variant == "dense" else n_moe)
            assert out["final_loss"] == out["final_loss"] and out["step_ms"] > 0
