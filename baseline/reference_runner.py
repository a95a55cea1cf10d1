"""Runs the UNMODIFIED reference package (baseline/_ref/data_pipeline) on the headline configuration.

Only the reference's public API is used: `SOTAConfig.from_dict`, `SOTATrainer(config)`,
`.setup_model(model=<random-init HF LlamaForCausalLM>)`, `.train(dataloader)`.  Timing is taken by the dataloader
object handed to `train()`: it records a CUDA event (after a barrier + synchronize) right before it yields the first
timed batch and another one when the loop asks for the batch after the last, so the timed region is exactly K of
the reference's own steps, including its host->device copies and host syncs.  None of this framework's models,
kernels or engines are imported here.
"""
from __future__ import annotations

import json
import os
import sys
import traceback
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"
ROOT = Path(__file__).resolve().parent.parent

SHAPES = {
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=8192),
    "tiny": dict(vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=4,
                 num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=8192),
}


class TimedBatches:
    def __init__(self, batches, warmup, world):
        import torch
        self.batches, self.warmup, self.world = batches, warmup, world
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)
        self.sampler = None
        self.clocks = None

    def __len__(self):
        return len(self.batches)

    def _fence(self):
        import torch
        import torch.distributed as dist
        if self.world > 1 and dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    def __iter__(self):
        for i, b in enumerate(self.batches):
            if i == self.warmup:
                self._fence()
                if self.sampler is not None:
                    self.sampler.start()
                self.e0.record()
            yield b
        self.e1.record()
        self._fence()
        if self.sampler is not None:
            self.clocks = self.sampler.stop()


def _attempt(args, world, rank, local, use_kernels: bool, grad_ckpt: bool):
    import torch
    import torch.distributed as dist
    from transformers import LlamaConfig, LlamaForCausalLM

    sys.path.insert(0, str(REF_DIR))
    from data_pipeline.trainer.core.sota_config import SOTAConfig
    from data_pipeline.trainer.trainers.sota_trainer import SOTATrainer

    seq, mb = args.seq, args.micro_batch
    try:
        import flash_attn  # noqa: F401
        attn = "flash_attention_2"
    except Exception:
        attn = "sdpa"
    raw = {
        "training_mode": "full",
        "model": {"name_or_path": "random-init-llama", "torch_dtype": "bfloat16", "attn_implementation": attn},
        "lora": {"enabled": False},
        "optimizer": {"type": "adamw", "learning_rate": 2e-5, "weight_decay": 0.01, "max_grad_norm": 1.0},
        "scheduler": {"type": "cosine", "warmup_steps": 0, "warmup_ratio": 0.0},
        "loss": {"type": "cross_entropy"},
        "distributed": {"enabled": world > 1, "backend": "nccl", "strategy": "fsdp2", "world_size": world,
                        "gradient_checkpointing": grad_ckpt,
                        "fsdp_config": {"sharding_strategy": "full_shard", "mixed_precision": "bf16",
                                        "activation_checkpointing": grad_ckpt, "gradient_accumulation_steps": 1,
                                        "gradient_clipping_norm": 1.0, "use_triton_kernels": use_kernels}},
        "hardware": {"device": "cuda", "precision": "bf16", "compile_model": False},
        "kernels": {"use_triton": use_kernels, "use_flash_attention": True, "use_fused_rope": use_kernels,
                    "use_fused_rms_norm": use_kernels, "use_fused_cross_entropy": use_kernels,
                    "activation_checkpointing": grad_ckpt},
        "data": {"max_seq_length": seq},
        "training": {"output_dir": "/tmp/ts_ref_out", "num_train_epochs": 1, "max_steps": -1,
                     "per_device_train_batch_size": mb, "gradient_accumulation_steps": 1, "eval_strategy": "no",
                     "save_strategy": "no", "save_steps": 10 ** 9, "logging_steps": 10 ** 9, "seed": 42},
    }
    cfg = SOTAConfig.from_dict(raw)
    trainer = SOTATrainer(cfg)
    torch.manual_seed(0)
    hf_cfg = LlamaConfig(**SHAPES[args.model], attn_implementation=attn, use_cache=False,
                         tie_word_embeddings=False)
    with torch.device("cuda", local):
        model = LlamaForCausalLM(hf_cfg).to(torch.bfloat16)
    trainer.setup_model(model=model)
    g = torch.Generator().manual_seed(1234 + rank)
    n = args.warmup + args.steps
    batches = []
    for _ in range(n):
        ids = torch.randint(0, hf_cfg.vocab_size, (mb, seq), generator=g, dtype=torch.int64).pin_memory()
        batches.append({"input_ids": ids, "attention_mask": torch.ones_like(ids).pin_memory(), "labels": ids})
    timed = TimedBatches(batches, args.warmup, world)
    if rank == 0:
        sys.path.insert(0, str(ROOT))
        from bench import ClockSampler
        timed.sampler = ClockSampler(local)
    trainer.train(timed)
    ms = timed.e0.elapsed_time(timed.e1)
    t = torch.tensor([ms], device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    steps_done = int(getattr(trainer.state, "global_step", n))
    return float(t.item()), timed.clocks, attn, steps_done, batches[0]["input_ids"].numel() * 8 * 2


def run(args) -> dict:
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    errors = []
    # prefer the reference's own defaults (its kernels on, no recompute); fall back to settings it also ships
    for use_kernels, ckpt in ((True, False), (True, True), (False, False), (False, True)):
        try:
            ms, clocks, attn, steps_done, h2d = _attempt(args, world, rank, local, use_kernels, ckpt)
            if steps_done < args.warmup + args.steps:
                raise RuntimeError(f"reference completed {steps_done} of {args.warmup + args.steps} steps "
                                   f"(it skipped steps)")
            tokens = args.micro_batch * args.seq * world * args.steps
            value = tokens / (ms / 1e3)
            out = {"impl": "reference", "metric": "train tokens/s/box (Llama-3-8B FSDP2 bf16)", "value": value,
                   "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                   "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                   "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
                   "config": {"model": args.model, "global_batch": args.micro_batch * world, "seq_len": args.seq,
                              "parallelism": f"fsdp{world}" if world > 1 else "single", "attention": attn,
                              "reference_kernels": use_kernels, "activation_checkpointing": ckpt,
                              "l2": "inputs larger than L2"},
                   "clocks": clocks,
                   "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                           "d2h_bytes_per_step": 8 * world},
                   "gpu_launches": None, "fallbacks_tried": errors}
            return out if rank == 0 else {}
        except Exception as e:   # noqa: BLE001
            errors.append(f"kernels={use_kernels} ckpt={ckpt}: {type(e).__name__}: {str(e)[:200]}")
            if os.environ.get("TS_REF_DEBUG"):
                traceback.print_exc()
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            if world > 1:
                break   # a failed multi-rank attempt leaves collectives in an unknown state: do not retry in-process
    return {"impl": "reference", "unavailable": "reference run failed: " + " | ".join(errors)[:600]} if rank == 0 else {}


def run_reference(args) -> dict:
    """Entry point of `bench.py --impl reference`."""
    if not (REF_DIR / "data_pipeline").exists():
        return {"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"}
    return run(args)
