"""Sharded checkpoints in the torch.distributed.checkpoint directory format (the reference's `dcp_save` layout)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from trainscale_b200.ckpt.dcp import is_dcp_checkpoint, load_dcp_checkpoint, save_dcp_checkpoint
from trainscale_b200.models.llama import LlamaConfig, build_model
from trainscale_b200.parallel.flat_engine import EngineConfig, FlatShardedEngine

CFG = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=16)


def _trained(seed=1):
    model = build_model(CFG, dtype=torch.float32, device="cpu", seed=seed)
    eng = FlatShardedEngine(model, EngineConfig(param_dtype=torch.float32, lr=1e-2), device=torch.device("cpu"))
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(0))
    for _ in range(2):
        eng.backward(model(ids, labels=ids).loss)
        eng.step()
    return model, eng


def test_single_process_roundtrip_and_plain_dcp_reader(tmp_path):
    import torch.distributed.checkpoint as dcp
    model, eng = _trained()
    save_dcp_checkpoint(eng, model, tmp_path / "ck", epoch=0, step=2)
    assert is_dcp_checkpoint(tmp_path / "ck")
    meta = torch.load(tmp_path / "ck" / "meta.pt", weights_only=False)
    assert meta["api_version"] == "dcp_modern_v2" and meta["config"]["world_size"] == 1
    # any DCP reader sees HuggingFace parameter names under "model." and AdamW state under "optimizer.state."
    keys = set(dcp.FileSystemReader(str(tmp_path / "ck")).read_metadata().state_dict_metadata)
    q = "model.model.layers.0.self_attn.q_proj.weight"
    assert q in keys and "model.lm_head.weight" in keys and "model.model.layers.1.mlp.up_proj.weight" in keys
    assert "optimizer.state.model.layers.0.self_attn.q_proj.weight.exp_avg_sq" in keys
    plain = {"model": {"model.layers.0.self_attn.q_proj.weight": torch.zeros(64, 64)}}
    dcp.load(plain, storage_reader=dcp.FileSystemReader(str(tmp_path / "ck")), no_dist=True)
    want = model.model.layers[0].self_attn.wqkv.detach()[:64]
    assert torch.equal(plain["model"]["model.layers.0.self_attn.q_proj.weight"], want)
    # and back into a fresh engine
    fresh = build_model(CFG, dtype=torch.float32, device="cpu", seed=7)
    e2 = FlatShardedEngine(fresh, EngineConfig(param_dtype=torch.float32, lr=1e-2), device=torch.device("cpu"))
    load_dcp_checkpoint(e2, fresh, tmp_path / "ck")
    for (n, p), (_, q_) in zip(fresh.named_parameters(), model.named_parameters()):
        assert torch.equal(p, q_), n
    for u, v in zip(e2.units, eng.units):
        assert torch.equal(u.exp_avg, v.exp_avg) and torch.equal(u.exp_avg_sq, v.exp_avg_sq) and torch.equal(u.master, v.master)
    assert e2.step_count == 2
    # both continue identically
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(5))
    for m, e in ((model, eng), (fresh, e2)):
        e.backward(m(ids, labels=ids).loss)
        e.step()
    for (n, p), (_, q_) in zip(fresh.named_parameters(), model.named_parameters()):
        assert torch.equal(p, q_), n


@pytest.mark.parametrize("strategy,port", [("FULL_SHARD", 29691), ("SHARD_GRAD_OP", 29692)])
def test_two_rank_save_single_process_load(tmp_path, strategy, port):
    case = Path(__file__).parent / "dist_cases" / "dcp_roundtrip.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(case), "--strategy", strategy, "--dir", str(tmp_path / "ck")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert f"RESULT dcp strategy={strategy} ok=True" in r.stdout


def test_trainer_writes_and_resumes_dcp_checkpoints(tmp_path):
    """`distributed.fsdp_config.checkpoint_format: dcp`: the trainer's checkpoint directory is a DCP directory, it
    passes verification, and a new trainer resumes weights, optimizer state and step from it."""
    from trainscale_b200.ckpt import verify_checkpoint
    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.trainer.sota_trainer import SOTATrainer

    def make():
        return SOTATrainer(SOTAConfig.from_dict({
            "model": {"architecture": {"vocab_size": 128, "hidden_size": 64, "intermediate_size": 96, "num_hidden_layers": 2,
                                       "num_attention_heads": 4, "num_key_value_heads": 2}},
            "optimizer": {"type": "adamw", "learning_rate": 1e-2}, "scheduler": {"type": "constant", "warmup_steps": 0},
            "distributed": {"enabled": False, "strategy": "fsdp2", "fsdp_config": {"checkpoint_format": "dcp"}},
            "hardware": {"device": "cpu", "precision": "fp32"}, "data": {"max_seq_length": 16},
            "training": {"output_dir": str(tmp_path), "max_steps": 3, "save_strategy": "no", "eval_strategy": "no"}}))
    tr = make()
    tr.setup_model()
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(0))
    for _ in range(3):
        tr.train_step({"input_ids": ids, "labels": ids})
    ck = tr.save_checkpoint()
    assert is_dcp_checkpoint(ck) and (ck / "trainer_state.pt").exists() and not (ck / "optim").exists()
    assert verify_checkpoint(ck) == []
    tr2 = make()
    tr2.setup_model()
    tr2.setup_optimizer()
    tr2.setup_scheduler(3)
    tr2.load_checkpoint(ck)
    for (n, p), (_, q) in zip(tr2.model.named_parameters(), tr.model.named_parameters()):
        assert torch.equal(p, q), n
    assert tr2.state.global_step == 3 and tr2.engine.step_count == 3
    assert torch.equal(tr2.engine.units[0].exp_avg_sq, tr.engine.units[0].exp_avg_sq)
