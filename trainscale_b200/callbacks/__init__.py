"""Training callbacks: the 11-hook protocol, a handler that actually fires them from SOTATrainer, and the stock
callbacks (early stopping, checkpointing, logging with console / TensorBoard / W&B backends, progress bar).

Hook names and stock callbacks follow data_pipeline/trainer/callbacks/__init__.py:61-634.  (The reference's
SOTATrainer registers callbacks but never triggers them, data_pipeline/trainer/trainers/sota_trainer.py:839-881;
here every hook is fired by the loop.)
"""
from __future__ import annotations

from enum import Enum

import json
import logging
import math
import os
import shutil
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..utils.refargs import ANY, reference_kwargs

logger = logging.getLogger("trainscale_b200")

HOOKS = ("on_init_end", "on_train_begin", "on_train_end", "on_epoch_begin", "on_epoch_end", "on_step_begin",
         "on_step_end", "on_evaluate", "on_save", "on_load", "on_log", "on_prediction_step")


@dataclass
class CallbackContext:
    trainer: Any = None
    state: Any = None
    config: Any = None
    model: Any = None
    optimizer: Any = None
    scheduler: Any = None
    metrics: dict = field(default_factory=dict)
    logs: dict = field(default_factory=dict)
    should_stop: bool = False
    should_save: bool = False
    should_evaluate: bool = False
    should_log: bool = False


class Callback:
    """Override any of the hooks; each receives the shared CallbackContext.  Callbacks run in ascending `order`
    (`priority` is the reference's name for the same number)."""
    order = 0
    trainer: Any = None

    def __init__(self, trainer=None):
        if trainer is not None:
            self.trainer = trainer

    @property
    def priority(self) -> int:
        return self.order

    def set_trainer(self, trainer) -> None:
        self.trainer = trainer

    def on_init_end(self, ctx): ...
    def on_train_begin(self, ctx): ...
    def on_train_end(self, ctx): ...
    def on_epoch_begin(self, ctx): ...
    def on_epoch_end(self, ctx): ...
    def on_step_begin(self, ctx): ...
    def on_step_end(self, ctx): ...
    def on_evaluate(self, ctx): ...
    def on_save(self, ctx): ...
    def on_load(self, ctx): ...
    def on_log(self, ctx): ...
    def on_prediction_step(self, ctx): ...


class CallbackHandler:
    def __init__(self, callbacks: list[Callback] | None = None):
        self.callbacks: list[Callback] = []
        for c in callbacks or []:
            self.add(c)

    @reference_kwargs(callback="cb")
    def add(self, cb: Callback | type) -> None:
        cb = cb() if isinstance(cb, type) else cb
        self.callbacks.append(cb)
        self.callbacks.sort(key=lambda c: c.order)

    @reference_kwargs(callback_type="cb_type")
    def remove(self, cb_type: type) -> None:
        if not isinstance(cb_type, type):                 # an instance: remove exactly that callback
            self.callbacks = [c for c in self.callbacks if c is not cb_type]
            return
        self.callbacks = [c for c in self.callbacks if not isinstance(c, cb_type)]

    def fire(self, hook: str, ctx: CallbackContext) -> CallbackContext:
        if hook not in HOOKS:
            raise ValueError(f"unknown hook {hook}")
        for c in self.callbacks:
            getattr(c, hook)(ctx)
        return ctx

    # the reference's method names (data_pipeline/trainer/callbacks/__init__.py:176-217)
    add_callback = add
    remove_callback = remove

    def set_trainer(self, trainer) -> None:
        for c in self.callbacks:
            if hasattr(c, "set_trainer"):
                c.set_trainer(trainer)

    def trigger(self, event: str, ctx: CallbackContext) -> CallbackContext:
        """Like `fire`, but later callbacks are skipped once one of them has set `ctx.should_stop`."""
        if event not in HOOKS:
            raise ValueError(f"unknown hook {event}")
        for c in self.callbacks:
            handler = getattr(c, event, None)
            if handler is not None:
                handler(ctx)
                if ctx.should_stop:
                    break
        return ctx

    def __getattr__(self, name):
        if name in HOOKS:
            return lambda ctx: self.fire(name, ctx)
        raise AttributeError(name)


class EarlyStoppingCallback(Callback):
    """Stops training after `patience` evaluations without an improvement of more than `threshold`.  The reference's
    names are taken too: `monitor` (metric), `min_delta` (threshold), `mode` = "min" | "max" (greater_is_better) and
    `restore_best`, which keeps a host copy of the best weights and loads it back when training ends."""

    @reference_kwargs(monitor="metric", min_delta="threshold")
    def __init__(self, patience: int = 3, threshold: float = 0.0, metric: str = "eval_loss", greater_is_better=False,
                 mode: str | None = None, restore_best: bool = False):
        if mode is not None:
            if mode not in ("min", "max"):
                raise ValueError("mode must be 'min' or 'max'")
            greater_is_better = mode == "max"
        self.patience, self.threshold, self.metric, self.greater = patience, threshold, metric, greater_is_better
        self.restore_best, self.best_state = restore_best, None
        self.best: float | None = None
        self.counter = 0

    def on_train_end(self, ctx):
        if self.restore_best and self.best_state is not None and ctx.model is not None:
            ctx.model.load_state_dict(self.best_state)

    def on_evaluate(self, ctx):
        v = ctx.metrics.get(self.metric)
        if v is None:
            return
        improved = self.best is None or ((v > self.best + self.threshold) if self.greater
                                         else (v < self.best - self.threshold))
        if improved:
            self.best, self.counter = v, 0
            if self.restore_best and ctx.model is not None:
                self.best_state = {k: t.detach().to("cpu", copy=True) for k, t in ctx.model.state_dict().items()}
        else:
            self.counter += 1
            if self.counter >= self.patience:
                ctx.should_stop = True


class CheckpointCallback(Callback):
    """save_strategy steps | epoch | best, rotation by save_total_limit (checkpoint-best is never pruned)."""

    @reference_kwargs(save_dir="output_dir")
    def __init__(self, output_dir: str, save_strategy: str = "steps", save_steps: int = 100, save_total_limit: int = 3,
                 metric: str = "eval_loss", greater_is_better: bool = False, config=None):
        """`config`: a checkpoint configuration object (`save_strategy`, `save_steps`, `save_total_limit`,
        `metric_for_best_model`, `greater_is_better`) whose attributes replace the keyword defaults."""
        if config is not None:
            save_strategy = getattr(config, "save_strategy", save_strategy)
            save_strategy = getattr(save_strategy, "value", save_strategy)
            save_steps = getattr(config, "save_steps", save_steps)
            save_total_limit = getattr(config, "save_total_limit", save_total_limit)
            metric = getattr(config, "metric_for_best_model", metric) or metric
            greater_is_better = getattr(config, "greater_is_better", greater_is_better)
        self.output_dir, self.strategy, self.save_steps = Path(output_dir), save_strategy, save_steps
        self.limit, self.metric, self.greater = save_total_limit, metric, greater_is_better
        self.best = None

    def on_step_end(self, ctx):
        if self.strategy == "steps" and self.save_steps > 0 and ctx.state.global_step % self.save_steps == 0:
            ctx.should_save = True

    def on_epoch_end(self, ctx):
        if self.strategy in ("epoch", "epochs"):
            ctx.should_save = True

    def on_evaluate(self, ctx):
        if self.strategy != "best":
            return
        v = ctx.metrics.get(self.metric)
        if v is not None and (self.best is None or (v > self.best if self.greater else v < self.best)):
            self.best = v
            ctx.should_save = True

    def on_save(self, ctx):
        self.cleanup_old_checkpoints()

    def cleanup_old_checkpoints(self):
        if self.limit is None or self.limit <= 0 or not self.output_dir.exists():
            return
        ckpts = []
        for p in self.output_dir.glob("checkpoint-*"):
            tail = p.name.split("-", 1)[1]
            if tail.isdigit():
                ckpts.append((int(tail), p))
        ckpts.sort()
        for _, p in ckpts[:-self.limit]:
            shutil.rmtree(p, ignore_errors=True)


class LoggingBackend(str, Enum):
    CONSOLE = "console"
    TENSORBOARD = "tensorboard"
    WANDB = "wandb"
    JSONL = "jsonl"


class LoggingCallback(Callback):
    def __init__(self, logging_steps: int = 10, backends: tuple[str, ...] = ("console",), log_dir: str | None = None,
                 rank: int = 0, config=None):
        """`config`: a logging configuration object (`logging_steps`, `report_to`, `logging_dir`)."""
        if config is not None:
            logging_steps = getattr(config, "logging_steps", logging_steps)
            backends = tuple(getattr(config, "report_to", backends) or backends)
            log_dir = getattr(config, "logging_dir", log_dir)
        self.logging_steps, self.backends, self.log_dir, self.rank = logging_steps, backends, log_dir, rank
        self._tb = None
        self._wandb = None
        self._jsonl = None

    def on_train_begin(self, ctx):
        if self.rank != 0:
            return
        if "tensorboard" in self.backends:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self._tb = SummaryWriter(self.log_dir)
            except Exception:   # tensorboard not installed
                self._tb = None
        if "wandb" in self.backends:
            try:
                import wandb
                self._wandb = wandb
            except Exception:
                self._wandb = None
        if "jsonl" in self.backends and self.log_dir:
            Path(self.log_dir).mkdir(parents=True, exist_ok=True)
            self._jsonl = open(Path(self.log_dir) / "train_log.jsonl", "a")

    def on_step_end(self, ctx):
        if self.logging_steps > 0 and ctx.state.global_step % self.logging_steps == 0:
            ctx.should_log = True

    def on_log(self, ctx):
        if self.rank != 0:
            return
        step = ctx.state.global_step
        if "console" in self.backends and ctx.logs.get("line"):
            logger.info(ctx.logs["line"])
        scalars = {k: v for k, v in ctx.logs.items() if isinstance(v, (int, float))}
        if self._tb is not None:
            for k, v in scalars.items():
                self._tb.add_scalar(k, v, step)
        if self._wandb is not None and getattr(self._wandb, "run", None) is not None:
            self._wandb.log(scalars, step=step)
        if self._jsonl is not None:
            self._jsonl.write(json.dumps({"step": step, **scalars}) + "\n")
            self._jsonl.flush()

    def on_train_end(self, ctx):
        if self._tb is not None:
            self._tb.close()
        if self._jsonl is not None:
            self._jsonl.close()


class ProgressCallback(Callback):
    def __init__(self, rank: int = 0, refresh_rate: int = 1):
        """`refresh_rate`: the bar is advanced every that many steps (by that many)."""
        self.rank, self.bar, self.refresh_rate, self._pending = rank, None, max(1, int(refresh_rate)), 0

    def on_train_begin(self, ctx):
        if self.rank == 0:
            try:
                from tqdm import tqdm
                self.bar = tqdm(total=getattr(ctx.state, "max_steps", None), desc="train", leave=False)
            except Exception:
                self.bar = None

    def on_step_end(self, ctx):
        if self.bar is not None:
            self._pending += 1
            if self._pending >= self.refresh_rate:
                self.bar.update(self._pending)
                self._pending = 0

    def on_train_end(self, ctx):
        if self.bar is not None:
            self.bar.update(self._pending)
            self.bar.close()
