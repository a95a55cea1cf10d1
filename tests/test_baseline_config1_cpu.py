"""Tiny Llama, CPU / gloo DDP world_size=2, YAML-configured, 20 steps: the loss curve goes down and both ranks end
with identical weights (the config is configs/llama_tiny_cpu_ddp.yaml, shortened sequences for test time)."""
import json
import subprocess
import sys
from pathlib import Path

import yaml

ROOT = Path(__file__).resolve().parent.parent


def test_tiny_llama_gloo_ddp_20_steps(tmp_path):
    raw = yaml.safe_load((ROOT / "configs" / "llama_tiny_cpu_ddp.yaml").read_text())
    raw["data"]["max_seq_length"] = 64
    raw["model"]["architecture"]["vocab_size"] = 512      # a vocabulary the 20 steps can make progress on
    raw["optimizer"]["learning_rate"] = 3e-3
    raw["data"]["dataset_config"] = "arith"             # learnable toy task: next token = token + 7 (mod V)
    raw["data"]["packing"] = False
    raw["training"]["per_device_train_batch_size"] = 4
    raw["training"]["output_dir"] = str(tmp_path / "out")
    cfg = tmp_path / "cfg.yaml"
    cfg.write_text(yaml.safe_dump(raw))
    res = tmp_path / "res.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29691", "-m", "trainscale_b200.train", "--config", str(cfg), "--json", str(res)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    out = json.loads(res.read_text())
    assert out["global_step"] == 20
    losses = out["losses"]
    assert len(losses) == 4 and losses[-1] < losses[0] - 0.5, losses


def test_config1_unmodified_matches_a_plain_pytorch_run(tmp_path):
    """configs/llama_tiny_cpu_ddp.yaml exactly as shipped (4 layers, d 256, vocab 32000, packed sequences of 512
    uniform-random tokens, 8 per rank, AdamW 3e-4 with cosine schedule, 20 steps) on two gloo ranks, against the same
    model trained in this process with torch.optim.AdamW on the concatenated batches: the logged loss curve (window
    means at steps 5, 10, 15, 20) must agree, start near ln(32000) and stay finite."""
    import math
    import os

    import torch

    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.data.synthetic import synthetic_dataloader
    from trainscale_b200.models.llama import LlamaConfig, build_model
    from trainscale_b200.schedulers import create_scheduler

    cfg_path = ROOT / "configs" / "llama_tiny_cpu_ddp.yaml"
    res = tmp_path / "res.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29692", "-m", "trainscale_b200.train", "--config", str(cfg_path), "--json", str(res),
           "--set", f"training.output_dir={tmp_path / 'out'}"]
    env = dict(os.environ, OMP_NUM_THREADS="4")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = json.loads(res.read_text())["losses"]
    assert len(got) == 4 and all(math.isfinite(x) for x in got)
    assert abs(got[0] - math.log(32000)) < 0.6

    raw = yaml.safe_load(cfg_path.read_text())
    c = SOTAConfig.from_dict(raw)
    model = build_model(LlamaConfig.from_dict(raw["model"]["architecture"]), dtype=torch.float32, device="cpu",
                        seed=c.training.seed)
    opt = torch.optim.AdamW(model.parameters(), lr=c.optimizer.learning_rate, betas=tuple(c.optimizer.betas),
                            eps=c.optimizer.eps, weight_decay=c.optimizer.weight_decay)
    sched = create_scheduler(opt, "cosine", 20, warmup_steps=c.scheduler.warmup_steps, warmup_ratio=0.0,
                             min_lr_ratio=c.scheduler.min_lr_ratio)
    loaders = [iter(synthetic_dataloader(32000, 512, 8, num_batches=20, seed=c.data.seed, packed=True, rank=rk))
               for rk in range(2)]
    window, want = [], []
    for step in range(20):
        batches = [next(it) for it in loaders]
        losses = []
        opt.zero_grad(set_to_none=True)
        for b in batches:      # the mean of the two ranks' mean losses, as data parallelism averages them
            out = model(input_ids=b["input_ids"], labels=b["labels"], attention_mask=b["attention_mask"],
                        position_ids=b["position_ids"], doc_ids=b["document_ids"])
            (out.loss / 2).backward()
            losses.append(float(out.loss.detach()))
        torch.nn.utils.clip_grad_norm_(model.parameters(), c.optimizer.max_grad_norm)
        opt.step()
        sched.step()
        window.append(sum(losses) / 2)
        if (step + 1) % 5 == 0:
            want.append(sum(window) / len(window))
            window = []
    for a, b in zip(got, want):
        assert abs(a - b) < 5e-3, (got, want)
