"""The transformers / TRL side of the fused head on CPU: routing rules with their reasons, the
causal-LM forward's hand-over to the installed forward, and TRL's three metrics computed from the
per-token terms with a stand-in trainer (the reference covers these with TRL installed,
tests_local/test_lm_head_trainer.py; TRL is not in this image)."""

import types

import torch

from claudemaxing_b200 import lm_head_loss as L
from claudemaxing_b200 import trainer_glue as G


class _Accelerator:
    def gather_for_metrics(self, t):      # two identical ranks
        return torch.stack([t, t])


def _trainer(**over):
    tr = types.SimpleNamespace(
        model=types.SimpleNamespace(training=True), args=types.SimpleNamespace(n_gpu=1),
        accelerator=_Accelerator(), _total_train_tokens=0,
        _metrics={"train": {"entropy": [], "num_tokens": [], "mean_token_accuracy": []}})
    for k, v in over.items():
        setattr(tr, k, v)
    return tr


def test_trainer_rules_name_the_reason():
    model = torch.nn.Linear(2, 2)
    inputs = {"labels": torch.zeros(1, 2, dtype=torch.long)}
    assert G.explain_trainer_route(_trainer(), "not a module", inputs)[1].startswith("not a training step")
    assert "several GPUs" in G.explain_trainer_route(
        _trainer(args=types.SimpleNamespace(n_gpu=2)), model, inputs)[1]
    assert "labels" in G.explain_trainer_route(_trainer(), model, {"input_ids": None})[1]
    assert G.explain_trainer_route(_trainer(label_smoother=object()), model, inputs)[1] == "label smoothing"
    assert G.explain_trainer_route(_trainer(compute_loss_func=len), model, inputs)[1] == "custom loss function"
    # every rule passes, but the model is not a patched causal LM
    lm, why = G.explain_trainer_route(_trainer(), model, inputs)
    assert lm is None and "patched" in why


def test_batch_rules_name_the_reason():
    lm = types.SimpleNamespace(lm_head=torch.nn.Linear(4, 8, bias=False),
                               config=types.SimpleNamespace(_attn_implementation="sdpa"))
    ids = torch.zeros(2, 3, dtype=torch.long)
    assert "CUDA" in G.explain_batch_route(lm, {"input_ids": ids}, ids)      # CPU batch: not packed
    assert G._pack_batch(lm, {"input_ids": ids, "attention_mask": torch.ones_like(ids)}, ids) is None


def test_metrics_follow_trl_definitions():
    tr = _trainer()
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    terms = L.StepTerms(token_loss=torch.zeros(2, 4),
                        token_entropy=torch.tensor([[1.0, 2.0, 3.0, 9.0], [4.0, 5.0, 9.0, 9.0]]),
                        correct=torch.tensor(3), labelled=torch.tensor(4))
    G._log_trl_metrics(tr, "train", {"attention_mask": mask}, terms)
    assert abs(tr._metrics["train"]["entropy"][0] - 3.0) < 1e-6          # (1+2+3+4+5)/5, padding masked
    assert tr._total_train_tokens == 10 and tr._metrics["train"]["num_tokens"] == [10]   # 5 x 2 ranks
    assert abs(tr._metrics["train"]["mean_token_accuracy"][0] - 0.75) < 1e-6
    # padding-free batches carry position_ids instead of a mask
    tr2 = _trainer()
    G._log_trl_metrics(tr2, "train", {"position_ids": torch.zeros(1, 7, dtype=torch.long)},
                       L.StepTerms(torch.zeros(1, 7), torch.ones(1, 7), torch.tensor(0), torch.tensor(0)))
    assert tr2._total_train_tokens == 14 and tr2._metrics["train"]["mean_token_accuracy"] == [0.0]
    try:
        G._log_trl_metrics(_trainer(), "train", {}, terms)
    except ValueError as err:
        assert "attention_mask" in str(err)
    else:
        raise AssertionError("inputs without mask or position ids must be refused")


def test_unflagged_forward_is_the_installed_one():
    import claudemaxing_b200 as solution
    from transformers import Qwen2Config, Qwen2ForCausalLM

    solution.apply()
    cfg = Qwen2Config(hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=4, num_key_value_heads=2, vocab_size=50)
    lm = Qwen2ForCausalLM(cfg)
    ids = torch.randint(0, 50, (2, 6))
    out = lm(input_ids=ids, labels=ids)                       # nobody asked for the fused head
    assert out.logits is not None and out.logits.shape == (2, 6, 50)
    lm.__dict__[L._REQUEST_ATTR] = True                       # asked, but a CPU model: logits path
    out = lm(input_ids=ids, labels=ids)
    assert out.logits is not None and torch.isfinite(out.loss)
    assert L._REQUEST_ATTR not in lm.__dict__                 # the flag is one-shot


def test_unpacked_puts_values_back_in_their_rows():
    ids = torch.tensor([[5, 6, 7, 0], [8, 9, 0, 0]])
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    p = G.pack_tokens(ids, mask, ids.clone())
    back = G._unpacked(torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0]), p)
    assert back.tolist() == [[1.0, 2.0, 3.0, 0.0], [4.0, 5.0, 0.0, 0.0]]
    pos = torch.tensor([[3, 4, 5, 0], [0, 1, 0, 0]])
    assert G.pack_tokens(ids, mask, ids.clone(), pos).pos.tolist() == [[3, 4, 5, 0, 1]]
    assert G.pack_tokens(ids, mask, ids.clone(), position_ids="auto") is None
