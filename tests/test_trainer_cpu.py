"""Single-process CPU training slice: YAML-shaped config -> SOTATrainer -> flat engine -> loss goes down,
checkpoint round-trip restores weights, optimizer shards and the step counter."""
import math

import torch

from trainscale_b200.config.sota_config import SOTAConfig
from trainscale_b200.data.synthetic import synthetic_dataloader
from trainscale_b200.trainer.sota_trainer import SOTATrainer

TINY = {"vocab_size": 512, "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2}


def make_cfg(tmp_path, **over):
    raw = {
        "training_mode": "full", "model": {"architecture": TINY},
        "optimizer": {"type": "adamw", "learning_rate": 3e-3, "weight_decay": 0.0},
        "scheduler": {"type": "cosine", "warmup_steps": 2, "warmup_ratio": 0.0, "min_lr_ratio": 0.1},
        "distributed": {"enabled": False, "strategy": "ddp", "gradient_checkpointing": False},
        "hardware": {"device": "cpu", "precision": "fp32"},
        "data": {"max_seq_length": 32},
        "training": {"output_dir": str(tmp_path), "num_train_epochs": 1, "max_steps": 12, "gradient_accumulation_steps": 2,
                     "per_device_train_batch_size": 4, "logging_steps": 4, "save_steps": 0, "save_strategy": "no",
                     "eval_strategy": "no", "early_stopping_patience": 0, "seed": 7},
    }
    for k, v in over.items():
        raw[k].update(v)
    return SOTAConfig.from_dict(raw)


def fixed_loader(n=64):
    # a tiny repeating corpus so that the model can actually fit it
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 512, (8, 32), generator=g)
    batches = [{"input_ids": base[i % 2 * 4:(i % 2) * 4 + 4], "attention_mask": torch.ones(4, 32, dtype=torch.long),
                "labels": base[i % 2 * 4:(i % 2) * 4 + 4]} for i in range(n)]
    return batches


def test_loss_decreases_and_logs(tmp_path):
    tr = SOTATrainer(make_cfg(tmp_path))
    tr.setup_model()
    out = tr.train(fixed_loader(24))
    hist = out["history"]
    assert out["global_step"] == 12
    assert hist[-1]["loss"] < hist[0]["loss"] - 0.3
    assert all(math.isfinite(h["grad_norm"]) for h in hist)


def test_checkpoint_roundtrip(tmp_path):
    tr = SOTATrainer(make_cfg(tmp_path))
    tr.setup_model()
    tr.train(fixed_loader(12))
    ck = tr.save_checkpoint()
    assert (ck / "trainer_state.pt").exists() and (ck / "meta.pt").exists()
    ref = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    m_ref = tr.engine.units[0].exp_avg.clone()
    tr2 = SOTATrainer(make_cfg(tmp_path))
    tr2.setup_model()
    tr2.setup_optimizer()
    tr2.setup_scheduler(12)
    tr2.load_checkpoint(ck)
    for n, p in tr2.model.named_parameters():
        assert torch.equal(p, ref[n]), n
    assert torch.equal(tr2.engine.units[0].exp_avg, m_ref)
    assert tr2.state.global_step == tr.state.global_step
    assert tr2.engine.step_count == tr.engine.step_count


def test_synthetic_packed_batch_schema():
    dl = synthetic_dataloader(1000, 128, 2, num_batches=2, packed=True, min_doc=16, max_doc=64)
    b = next(iter(dl))
    assert set(b) >= {"input_ids", "attention_mask", "labels", "document_ids", "position_ids"}
    d, p = b["document_ids"][0], b["position_ids"][0]
    starts = torch.nonzero(p == 0).flatten()
    assert starts[0] == 0 and torch.all(d[starts[1:]] == d[starts[1:] - 1] + 1)


def test_op_selective_recompute_matches_plain_path_on_cpu():
    """The operator-level recompute blocks fall back to the separate ops off the CUDA bf16 path: same loss and grads."""
    import torch
    from trainscale_b200.models.llama import LlamaConfig, build_model
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16)
    m = build_model(cfg, dtype=torch.float32, device="cpu", seed=0).train()
    ids = torch.randint(0, 128, (2, 24), generator=torch.Generator().manual_seed(0))
    l0 = m(input_ids=ids, labels=ids).loss
    l0.backward()
    g0 = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad(set_to_none=True)
    m.op_selective_recompute(True)
    l1 = m(input_ids=ids, labels=ids).loss
    l1.backward()
    assert abs(l0.item() - l1.item()) < 1e-6
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, g0[n], atol=1e-6), n


def test_numerical_stability_check_counts_bad_windows():
    from trainscale_b200.core.errors import GradientOverflowError
    from trainscale_b200.trainer.sota_trainer import SOTATrainer
    t = SOTATrainer.__new__(SOTATrainer)
    assert t._check_numerical_stability(1.0, 2.0, 3) is True
    assert t._check_numerical_stability(float("nan"), 2.0, 4) is False
    assert t._check_numerical_stability(1.0, 1e7, 5) is True and t._bad_windows == 0      # exploding only warns
    t.max_nonfinite_windows = 2
    assert t._check_numerical_stability(1.0, float("inf")) is False
    import pytest
    with pytest.raises(GradientOverflowError):
        t._check_numerical_stability(float("inf"))


def test_partial_accumulation_window_at_epoch_end_is_dropped(tmp_path):
    """A loader whose length is not a multiple of the accumulation steps: the left-over micro-batch of an epoch makes
    no step and must not leak into the next epoch's first update (the run equals one over the loader without it)."""
    def run(n_batches, sub):
        cfg = make_cfg(tmp_path / sub, training={"num_train_epochs": 2, "max_steps": 0, "gradient_accumulation_steps": 2})
        tr = SOTATrainer(cfg)
        tr.setup_model()
        out = tr.train(fixed_loader(8)[:n_batches])
        return out, {n: p.detach().clone() for n, p in tr.model.named_parameters()}, tr
    out5, p5, tr5 = run(5, "a")
    out4, p4, _ = run(4, "b")
    assert out5["global_step"] == out4["global_step"] == 4
    for n in p4:
        assert torch.equal(p5[n], p4[n]), n
    assert tr5.engine.micro_step % 2 == 0
