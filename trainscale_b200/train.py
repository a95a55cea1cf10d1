"""`python -m trainscale_b200.train --config X.yaml [--max-steps N] [--dry-run] [--verify]`

One YAML drives both halves: the data keys build a DataPipeline (or, with `dataset.name: synthetic`, the synthetic
packed-token loader) and the training keys build a SOTATrainer.  Under torchrun every rank runs this script.
Flags mirror the reference demos (data_pipeline/examples/rocm_sota_demo_fsdp2.py: --config / --verify / --dry-run /
--max-steps).
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
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(message)s")
    from .config.sota_config import SOTAConfig
    from .data.synthetic import synthetic_dataloader, synthetic_preference_dataloader
    from .trainer.sota_trainer import SOTATrainer

    raw = yaml.safe_load(open(a.config)) or {}
    cfg = SOTAConfig.from_dict(raw)
    if a.max_steps is not None:
        cfg.training.max_steps = a.max_steps
    if a.verify:
        cfg.training.max_steps = 1
    trainer = SOTATrainer(cfg)
    trainer.setup_model()
    ds = raw.get("dataset") or {}
    steps = cfg.training.max_steps if cfg.training.max_steps > 0 else 100
    if str(ds.get("name", "synthetic")).lower() == "synthetic" and trainer.preference_kind is not None:
        # preference objectives train on prompt / chosen / rejected triples: half of max_seq_length each for the
        # prompt and the response unless the dataset section says otherwise
        vocab = trainer.model.config.vocab_size
        p_len = int(ds.get("prompt_length", cfg.data.max_seq_length // 2))
        r_len = int(ds.get("response_length", cfg.data.max_seq_length - p_len))
        dl = synthetic_preference_dataloader(vocab, p_len, r_len, cfg.training.per_device_train_batch_size,
                                             num_batches=steps * cfg.training.gradient_accumulation_steps,
                                             seed=cfg.data.seed, rank=trainer.rank,
                                             pin_memory=trainer.device.type == "cuda")
        ev = None
    elif str(ds.get("name", "synthetic")).lower() == "synthetic":
        vocab = trainer.model.config.vocab_size
        dl = synthetic_dataloader(vocab, cfg.data.max_seq_length, cfg.training.per_device_train_batch_size,
                                  num_batches=steps * cfg.training.gradient_accumulation_steps, seed=cfg.data.seed,
                                  packed=cfg.data.packing, rank=trainer.rank, pin_memory=trainer.device.type == "cuda",
                                  mode=cfg.data.dataset_config or "uniform")
        ev = None
    else:
        from .data.pipeline import DataPipeline
        pipe = DataPipeline.from_config(raw).unwrap()
        dl = pipe.get_dataloader("train", cfg.training.per_device_train_batch_size, trainer.is_distributed, trainer.rank,
                                 trainer.world_size).unwrap()
        ev_r = pipe.get_dataloader("validation", cfg.training.per_device_eval_batch_size, trainer.is_distributed,
                                   trainer.rank, trainer.world_size)
        ev = ev_r.unwrap() if ev_r.is_ok() else None
    if a.dry_run:
        if trainer.is_main:
            print(json.dumps({"dry_run": True, "params": sum(p.numel() for p in trainer.model.parameters()),
                              "strategy": trainer.strategy, "world_size": trainer.world_size}))
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


if __name__ == "__main__":
    sys.exit(main())
