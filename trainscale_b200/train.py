"""`python -m trainscale_b200.train --config X.yaml [--max-steps N] [--dry-run] [--verify] [--set a.b=c ...]
[--measure K --measure-warmup W]`

One YAML drives both halves: the data keys build a DataPipeline (or, with `dataset.name: synthetic`, the synthetic
packed-token loader) and the training keys build a SOTATrainer.  Under torchrun every rank runs this script.
Flags mirror the reference demos (data_pipeline/examples/rocm_sota_demo_fsdp2.py: --config / --verify / --dry-run /
--max-steps).  `--set` overrides one key of the YAML (dotted path, YAML value), e.g. `--set distributed.comm=nccl`.
`--measure K` times K optimizer steps through `SOTATrainer.train_step` (host batches from the loader, loss read back
every step) after W warm-up steps, with CUDA events between a barrier + synchronize on both sides, takes the maximum
over ranks and prints one JSON line with tokens/s of the whole job, ms/step and peak memory.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys

import yaml


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--max-steps", type=int, default=None)
    ap.add_argument("--dry-run", action="store_true", help="build everything, run no step")
    ap.add_argument("--verify", action="store_true", help="one step + checkpoint round trip")
    ap.add_argument("--json", default=None, help="write the result summary here (rank 0)")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE", help="override a config key")
    ap.add_argument("--measure", type=int, default=0, help="time this many steps on the device and print one JSON line")
    ap.add_argument("--measure-warmup", type=int, default=2)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(message)s")
    from .config.sota_config import SOTAConfig
    from .data.synthetic import synthetic_dataloader, synthetic_preference_dataloader
    from .trainer.sota_trainer import SOTATrainer

    raw = yaml.safe_load(open(a.config)) or {}
    for item in a.set:
        key, _, val = item.partition("=")
        node = raw
        parts = key.split(".")
        for p_ in parts[:-1]:
            node = node.setdefault(p_, {})
        node[parts[-1]] = yaml.safe_load(val)
    cfg = SOTAConfig.from_dict(raw)
    if a.max_steps is not None:
        cfg.training.max_steps = a.max_steps
    if a.verify:
        cfg.training.max_steps = 1
    trainer = SOTATrainer(cfg)
    trainer.setup_model()
    ds = raw.get("dataset") or {}
    steps = cfg.training.max_steps if cfg.training.max_steps > 0 else 100
    if a.measure:
        steps = a.measure + a.measure_warmup
    if str(ds.get("name", "synthetic")).lower() == "synthetic" and trainer.preference_kind is not None:
        # preference objectives train on prompt / chosen / rejected triples: half of max_seq_length each for the
        # prompt and the response unless the dataset section says otherwise
        vocab = trainer.model.config.vocab_size
        p_len = int(ds.get("prompt_length", cfg.data.max_seq_length // 2))
        r_len = int(ds.get("response_length", cfg.data.max_seq_length - p_len))
        dl = synthetic_preference_dataloader(vocab, p_len, r_len, cfg.training.per_device_train_batch_size,
                                             num_batches=steps * cfg.training.gradient_accumulation_steps,
                                             seed=cfg.data.seed, rank=trainer.data_rank(),
                                             pin_memory=trainer.device.type == "cuda")
        ev = None
    elif str(ds.get("name", "synthetic")).lower() == "synthetic":
        vocab = trainer.model.config.vocab_size
        dl = synthetic_dataloader(vocab, cfg.data.max_seq_length, cfg.training.per_device_train_batch_size,
                                  num_batches=steps * cfg.training.gradient_accumulation_steps, seed=cfg.data.seed,
                                  packed=cfg.data.packing, rank=trainer.data_rank(), pin_memory=trainer.device.type == "cuda",
                                  mode=cfg.data.dataset_config or "uniform")
        ev = None
    else:
        from .data.pipeline import DataPipeline
        pipe = DataPipeline.from_config(raw).unwrap()
        dp = trainer._data_parallel_size()
        dl = pipe.get_dataloader("train", cfg.training.per_device_train_batch_size, dp > 1, trainer.data_rank(),
                                 dp).unwrap()
        ev_r = pipe.get_dataloader("validation", cfg.training.per_device_eval_batch_size, dp > 1,
                                   trainer.data_rank(), dp)
        ev = ev_r.unwrap() if ev_r.is_ok() else None
    if a.dry_run:
        if trainer.is_main:
            print(json.dumps({"dry_run": True, "params": sum(p.numel() for p in trainer.model.parameters()),
                              "strategy": trainer.strategy, "world_size": trainer.world_size}))
        trainer.cleanup()
        return 0
    if a.measure:
        summary = measure(trainer, dl, a.measure, a.measure_warmup, a.config, a.set)
        if trainer.is_main:
            print(json.dumps(summary), flush=True)
            if a.json:
                with open(a.json, "w") as f:
                    json.dump(summary, f)
        trainer.cleanup()
        return 0
    out = trainer.train(dl, ev)
    if a.verify:
        ck = trainer.save_checkpoint()
        trainer.load_checkpoint(ck)
    if trainer.is_main:
        summary = {k: v for k, v in out.items() if k != "history"}
        summary["losses"] = [h["loss"] for h in out["history"]]
        print(json.dumps(summary))
        if a.json:
            with open(a.json, "w") as f:
                json.dump(summary, f)
    trainer.cleanup()
    return 0


def measure(trainer, dl, steps: int, warmup: int, config_path: str, overrides: list) -> dict:
    """Device-timed throughput of `trainer.train_step` (see the module docstring)."""
    import torch
    import torch.distributed as dist
    it = iter(dl)
    dist_on = trainer.is_distributed
    cuda = trainer.device.type == "cuda"

    def fence():
        if dist_on:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    losses = []
    for _ in range(warmup):
        losses.append(trainer.train_step(next(it)))
    fence()
    if cuda:
        torch.cuda.reset_peak_memory_stats()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    import time
    t0 = time.perf_counter()
    tokens = 0
    for _ in range(steps):
        batch = next(it)
        tokens += trainer._batch_tokens(batch)
        losses.append(trainer.train_step(batch))
    if cuda:
        e1.record()
    fence()
    ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], device=trainer.device)
    if dist_on:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    global_tokens = tokens * trainer._data_parallel_size()      # ranks of one model replica see the same tokens
    out = {"config": config_path, "overrides": list(overrides), "world_size": trainer.world_size,
           "strategy": trainer.strategy, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
           "tokens_per_step": global_tokens // steps, "tokens_per_s": global_tokens / (ms / 1e3),
           "losses": [round(float(x), 4) for x in losses],
           "peak_mem_gb": (torch.cuda.max_memory_allocated() / 2 ** 30) if cuda else None,
           "timing": "CUDA events around the timed steps, barrier + synchronize on both sides, max over ranks"}
    eng = trainer.engine
    if eng is not None and hasattr(eng, "memory_summary"):
        out["memory"] = eng.memory_summary()
    try:
        from .parallel import tp_fused
        out["fused_tp_kernel_calls"] = dict(tp_fused.CALLS)
    except Exception:      # noqa: BLE001 - no CUDA libraries on this machine
        pass
    comm = getattr(trainer.config.distributed, "comm", None)
    out["comm"] = comm
    return out


if __name__ == "__main__":
    sys.exit(main())
