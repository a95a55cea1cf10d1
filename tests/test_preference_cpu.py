"""Preference training (DPO / SimPO / ORPO / KTO / CPO) selected from the config and driven by SOTATrainer."""
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

from trainscale_b200.config.sota_config import SOTAConfig
from trainscale_b200.data.synthetic import synthetic_preference_dataloader
from trainscale_b200.trainer.sota_trainer import SOTATrainer

TINY = {"vocab_size": 96, "hidden_size": 32, "intermediate_size": 64, "num_hidden_layers": 2,
        "num_attention_heads": 2, "num_key_value_heads": 1}


def make_cfg(tmp_path, loss=None, rl=None, mode="full", lr=5e-3, steps=12):
    raw = {"training_mode": mode, "model": {"architecture": TINY},
           "optimizer": {"type": "adamw", "learning_rate": lr, "weight_decay": 0.0},
           "scheduler": {"type": "constant", "warmup_steps": 0},
           "distributed": {"enabled": False, "strategy": "ddp"}, "hardware": {"device": "cpu", "precision": "fp32"},
           "data": {"max_seq_length": 16},
           "training": {"output_dir": str(tmp_path), "max_steps": steps, "num_train_epochs": 1, "logging_steps": 4,
                        "save_strategy": "no", "eval_strategy": "no", "per_device_train_batch_size": 4, "seed": 3,
                        "gradient_accumulation_steps": 1}}
    if loss:
        raw["loss"] = loss
    if rl:
        raw["rl"] = rl
    return SOTAConfig.from_dict(raw)


def seq_logp(model, ids, labels):
    """fp32 oracle: sum over response tokens of log softmax(logits)[next token]."""
    logits = model(input_ids=ids, return_logits=True).logits.float()
    lp = torch.log_softmax(logits[:, :-1], -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)
    m = (labels[:, 1:] != -100).float()
    return (lp * m).sum(-1), m.sum(-1)


def test_training_mode_rl_selects_the_preference_step(tmp_path):
    tr = SOTATrainer(make_cfg(tmp_path, rl={"enabled": True, "algorithm": "dpo"}, mode="rl"))
    assert tr.preference_kind == "dpo"
    assert SOTATrainer(make_cfg(tmp_path, loss={"type": "simpo"})).preference_kind == "simpo"
    assert SOTATrainer(make_cfg(tmp_path)).preference_kind is None


@pytest.mark.parametrize("kind", ["dpo", "simpo"])
def test_loss_equals_closed_form(tmp_path, kind):
    cfg = make_cfg(tmp_path, loss={"type": kind, "dpo_beta": 0.1, "simpo_gamma": 0.5})
    tr = SOTATrainer(cfg)
    tr.setup_model()
    batch = next(iter(synthetic_preference_dataloader(96, 8, 8, 4, num_batches=1)))
    loss, _ = tr._forward_loss(batch, 1.0)
    with torch.no_grad():
        pc, nc = seq_logp(tr.model, batch["chosen_input_ids"], batch["chosen_labels"])
        pr, nr = seq_logp(tr.model, batch["rejected_input_ids"], batch["rejected_labels"])
        if kind == "dpo":
            # the frozen reference is a copy of the initial policy: the reference terms cancel the policy's exactly
            rc, _ = seq_logp(tr.preference.ref, batch["chosen_input_ids"], batch["chosen_labels"])
            rr, _ = seq_logp(tr.preference.ref, batch["rejected_input_ids"], batch["rejected_labels"])
            want = -F.logsigmoid(0.1 * ((pc - pr) - (rc - rr))).mean()
            assert abs(float(want) - math.log(2.0)) < 1e-5
        else:
            want = -F.logsigmoid(0.1 * (pc / nc - pr / nr) - 0.5).mean()
    assert abs(float(loss) - float(want)) < 1e-5
    assert int(nc[0]) == 8        # the 8 response tokens; the prompt is masked


def test_dpo_reward_accuracy_moves_and_reference_stays_frozen(tmp_path):
    cfg = make_cfg(tmp_path, loss={"type": "dpo", "dpo_beta": 0.5}, lr=1e-2, steps=30)
    tr = SOTATrainer(cfg)
    tr.setup_model()
    ref0 = {n: p.detach().clone() for n, p in tr.preference.ref.named_parameters()}
    assert not any(p.requires_grad for p in tr.preference.ref.parameters())
    dl = synthetic_preference_dataloader(96, 8, 8, 4, num_batches=2)
    batches = list(dl) * 15                                   # a tiny corpus the policy can separate
    out = tr.train(batches)
    hist = out["history"]
    assert hist[0]["loss"] <= math.log(2.0) + 1e-3 and hist[-1]["loss"] < hist[0]["loss"] - 0.05
    assert hist[-1]["reward_accuracy"] >= 0.75 and hist[-1]["reward_margin"] > 0
    for n, p in tr.preference.ref.named_parameters():
        assert torch.equal(p, ref0[n]), n


@pytest.mark.parametrize("kind", ["orpo", "cpo", "kto"])
def test_other_objectives_step(tmp_path, kind):
    tr = SOTATrainer(make_cfg(tmp_path, loss={"type": kind}, steps=3))
    tr.setup_model()
    out = tr.train(list(synthetic_preference_dataloader(96, 8, 8, 4, num_batches=3)))
    assert out["global_step"] == 3 and math.isfinite(out["history"][-1]["loss"])


def test_config5_yaml_runs_from_the_cli_with_a_tiny_model(tmp_path):
    """configs/llama3_8b_dpo.yaml with the model swapped for a tiny one: the CLI builds preference batches for
    `dataset.name: synthetic` and trains the DPO objective."""
    import yaml
    root = Path(__file__).resolve().parent.parent
    raw = yaml.safe_load((root / "configs" / "llama3_8b_dpo.yaml").read_text())
    raw["model"] = {"architecture": TINY}
    raw["distributed"] = {"enabled": False, "strategy": "ddp", "gradient_checkpointing": True}
    raw["hardware"] = {"device": "cpu", "precision": "fp32"}
    raw["data"] = {"max_seq_length": 16}
    raw["training"].update(max_steps=2, per_device_train_batch_size=2, output_dir=str(tmp_path), logging_steps=1,
                           save_strategy="no")
    p = tmp_path / "dpo.yaml"
    p.write_text(yaml.safe_dump(raw))
    r = subprocess.run([sys.executable, "-m", "trainscale_b200.train", "--config", str(p), "--json", str(tmp_path / "o.json")],
                       capture_output=True, text=True, timeout=300, cwd=str(root))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    import json
    out = json.loads((tmp_path / "o.json").read_text())
    assert out["global_step"] == 2 and abs(out["losses"][0] - math.log(2.0)) < 1e-3


def test_two_rank_dpo_with_sharded_frozen_reference_matches_single_process():
    case = Path(__file__).parent / "dist_cases" / "preference_equivalence.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29681", str(case)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT preference strategy=FULL_SHARD" in r.stdout and "ok=True" in r.stdout
