"""Host-side failure cases (gloo / CPU; no GPU is involved, nothing is faulted on a device).

  --mode heartbeat   rank 2's heartbeats stop reaching the store from step 3 on; every rank notices within the timeout
  --mode exit        rank 1 leaves the job between steps; rank 0's next collective ends with an error (short timeout)
  --mode train       2-rank sharded training that checkpoints every step and dies at step 3 (injected exception)
  --mode resume      restart (any world size) from the newest undamaged checkpoint, finish, compare with an
                     uninterrupted single-process run
"""
import argparse
import datetime
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from trainscale_b200.parallel.dist_utils import FaultInjector, HeartbeatMonitor, InjectedFault  # noqa: E402

TOTAL_STEPS, VOCAB, SEQ, PER_RANK = 6, 128, 16, 2


def heartbeat_case():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    store = dist.distributed_c10d._get_default_store()
    mon = HeartbeatMonitor(store, rank, world)
    inj = FaultInjector("mute@3:rank2", rank)
    detected = None
    for step in range(160):
        inj.at_step(step)
        inj.beat(mon)
        time.sleep(0.05)
        stale = mon.stale_ranks(timeout_s=1.5)       # generous against scheduling hiccups of a loaded test machine
        if stale:
            detected = (step, stale)
            break
    print(f"RESULT rank={rank} detected={detected}", flush=True)
    ok = detected is not None and detected[1] == [2] and detected[0] >= 3
    time.sleep(1.0)          # let the others finish reading the store before the server rank leaves
    sys.exit(0 if ok else 1)


def exit_case():
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
    rank = dist.get_rank()
    inj = FaultInjector("exit@2:rank1", rank)
    t = torch.ones(4)
    try:
        for step in range(5):
            inj.at_step(step)            # rank 1 leaves here, between steps, with nothing in flight
            dist.all_reduce(t)
        print(f"RESULT rank={rank} finished (unexpected)", flush=True)
        sys.exit(1)
    except RuntimeError as e:
        print(f"RESULT rank={rank} collective failed at step {step}: {type(e).__name__}", flush=True)
        sys.exit(3)


def make_trainer(out_dir, world, enabled, resume=None):
    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.models.llama import LlamaConfig, build_model
    from trainscale_b200.trainer.sota_trainer import SOTATrainer
    cfg = SOTAConfig.from_dict({
        "training_mode": "full", "model": {"architecture": "llama-tiny"},
        "optimizer": {"type": "adamw", "learning_rate": 1e-2, "weight_decay": 0.0, "max_grad_norm": 1.0, "eps": 1e-3},
        "scheduler": {"type": "constant", "warmup_steps": 0}, "loss": {"type": "chunked_ce"},
        "distributed": {"enabled": enabled, "backend": "gloo", "strategy": "fsdp2" if enabled else "single",
                        "world_size": world, "gradient_checkpointing": False, "fsdp_sharding_strategy": "shard_grad_op"},
        "hardware": {"precision": "fp32", "device": "cpu"}, "data": {"max_seq_length": SEQ},
        "training": {"per_device_train_batch_size": PER_RANK, "gradient_accumulation_steps": 1, "max_steps": 100,
                     "logging_steps": 10 ** 9, "save_strategy": "no", "eval_strategy": "no", "output_dir": str(out_dir)}})
    mcfg = LlamaConfig(vocab_size=VOCAB, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    tr = SOTATrainer(cfg)
    tr.setup_model(model=build_model(mcfg, dtype=torch.float32, device="cpu", seed=7))
    tr.setup_optimizer()
    tr.setup_scheduler(100)
    return tr


def batch_for(step, rank, world, global_rows=4):
    g = torch.Generator().manual_seed(1000 + step)
    ids = torch.randint(0, VOCAB, (global_rows, SEQ), generator=g)
    per = global_rows // world
    mine = ids[rank * per:(rank + 1) * per]
    return {"input_ids": mine, "labels": mine}


def train_case(out_dir, fault):
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
    rank, world = dist.get_rank(), dist.get_world_size()
    tr = make_trainer(out_dir, world, True)
    inj = FaultInjector(fault, rank)
    try:
        for step in range(TOTAL_STEPS):
            inj.at_step(step)
            tr.train_step(batch_for(step, rank, world))
            tr.save_checkpoint()
            if rank == 0:
                print(f"step {step} saved checkpoint-{tr.state.global_step}", flush=True)
    except InjectedFault as e:
        print(f"RESULT rank={rank} died: {e}", flush=True)
        os._exit(5)              # the process is gone; its peers find out in their next collective
    print(f"RESULT rank={rank} finished", flush=True)


def resume_case(out_dir):
    from trainscale_b200.ckpt import find_latest_valid_checkpoint
    multi = int(os.environ.get("WORLD_SIZE", "1")) > 1
    if multi:
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    rank, world = (dist.get_rank(), dist.get_world_size()) if multi else (0, 1)
    skipped = []
    ck = find_latest_valid_checkpoint(Path(out_dir), log=skipped.append)
    tr = make_trainer(out_dir, world, multi)
    tr.load_checkpoint(ck)
    start = tr.state.global_step
    for step in range(start, TOTAL_STEPS):
        tr.train_step(batch_for(step, rank, world))
    # oracle: the same six steps without any interruption, one process
    saved = dist.is_initialized
    env_ws = os.environ.get("WORLD_SIZE")
    try:
        dist.is_initialized = lambda: False
        os.environ["WORLD_SIZE"] = "1"
        ref = make_trainer(Path(out_dir) / "oracle", 1, False)
        for step in range(TOTAL_STEPS):
            ref.train_step(batch_for(step, 0, 1))
    finally:
        dist.is_initialized = saved
        if env_ws is not None:
            os.environ["WORLD_SIZE"] = env_ws
    eng = tr.engine
    got = eng.full_model_state_dict() if eng is not None and hasattr(eng, "full_model_state_dict") else \
        dict(tr.model.named_parameters())
    want = dict(ref.model.named_parameters())
    worst = max(float((got[k].detach() - want[k].detach()).abs().max()) for k in want)
    ok = worst < 5e-4 and start >= 1
    if rank == 0:
        print(f"RESULT resumed_from={ck.name} start_step={start} skipped={len(skipped)} max|w-oracle|={worst:.2e} ok={ok}",
              flush=True)
    if multi:
        dist.barrier()
        dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", required=True, choices=["heartbeat", "exit", "train", "resume"])
    ap.add_argument("--out", default=None)
    ap.add_argument("--fault", default="")
    a = ap.parse_args()
    if a.mode == "heartbeat":
        heartbeat_case()
    elif a.mode == "exit":
        exit_case()
    elif a.mode == "train":
        train_case(a.out, a.fault)
    else:
        resume_case(a.out)
