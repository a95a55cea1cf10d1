"""Preference training on the CUDA kernels: per-token log-probs from the fused lm_head + log-prob kernel."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_dpo_step_on_gpu_matches_fp32_math(tmp_path):
    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.data.synthetic import synthetic_preference_dataloader
    from trainscale_b200.ops import _lib
    from trainscale_b200.trainer.sota_trainer import SOTATrainer

    arch = {"vocab_size": 1024, "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
            "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64}
    cfg = SOTAConfig.from_dict({
        "training_mode": "rl", "rl": {"enabled": True, "algorithm": "dpo"}, "loss": {"type": "dpo", "dpo_beta": 0.5},
        "model": {"architecture": arch}, "optimizer": {"type": "adamw", "learning_rate": 1e-3, "weight_decay": 0.0},
        "scheduler": {"type": "constant", "warmup_steps": 0},
        "distributed": {"enabled": False, "strategy": "fsdp2"}, "hardware": {"device": "cuda", "precision": "bf16"},
        "data": {"max_seq_length": 256},
        "training": {"output_dir": str(tmp_path), "max_steps": 4, "save_strategy": "no", "eval_strategy": "no",
                     "per_device_train_batch_size": 4, "gradient_accumulation_steps": 1, "logging_steps": 1}})
    tr = SOTATrainer(cfg)
    tr.setup_model()
    assert tr.preference_kind == "dpo" and tr.preference.ref is not None
    # make the reference differ from the policy, then check the loss against fp32 log-softmax math on both models
    with torch.no_grad():
        for p in tr.preference.ref.parameters():
            p.mul_(1.03)
    batch = {k: v.cuda() for k, v in next(iter(synthetic_preference_dataloader(1024, 128, 128, 4, num_batches=1))).items()}
    before = _lib.LAUNCHES
    loss, _ = tr._forward_loss(batch, 1.0)
    assert _lib.LAUNCHES > before

    def seq_logp(model, ids, labels):
        logits = model(input_ids=ids, return_logits=True).logits.float()
        lp = torch.log_softmax(logits[:, :-1], -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)
        return (lp * (labels[:, 1:] != -100).float()).sum(-1)

    with torch.no_grad():
        x = (seq_logp(tr.model, batch["chosen_input_ids"], batch["chosen_labels"]) -
             seq_logp(tr.model, batch["rejected_input_ids"], batch["rejected_labels"])) - \
            (seq_logp(tr.preference.ref, batch["chosen_input_ids"], batch["chosen_labels"]) -
             seq_logp(tr.preference.ref, batch["rejected_input_ids"], batch["rejected_labels"]))
        want = -F.logsigmoid(0.5 * x).mean()
    assert abs(float(loss) - float(want)) < 5e-2 * max(1.0, abs(float(want))), (float(loss), float(want))
    out = tr.train(list(synthetic_preference_dataloader(1024, 128, 128, 4, num_batches=4)))
    assert out["global_step"] == 4 and all(math.isfinite(h["loss"]) for h in out["history"])
    _lib.raise_on_any_device_error()
