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
