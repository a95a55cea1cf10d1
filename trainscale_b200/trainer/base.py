"""Legacy trainers: a generic `Trainer` over any nn.Module + torch optimizer (the loop that fires every callback),
and the specialised Pretraining / FineTuning / Seq2Seq / TextGeneration trainers.

After data_pipeline/trainer/base.py:129-834 and data_pipeline/trainer/trainers/__init__.py:28-388 (EMA weights and
curriculum sequence length in pre-training, layer-wise LR decay in fine-tuning, teacher-forced seq2seq loss, top-k /
top-p text generation).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..callbacks import CallbackContext, CallbackHandler
from ..config.training_args import TrainingArguments
from ..optim import clip_grad_norm_, create_optimizer
from ..schedulers import create_scheduler


class _State:
    def __init__(self):
        self.epoch, self.global_step, self.max_steps, self.best_metric = 0, 0, 0, float("inf")


class Trainer:
    def __init__(self, model: nn.Module, args: TrainingArguments | None = None, train_dataloader: Iterable | None = None,
                 eval_dataloader: Iterable | None = None, optimizer=None, scheduler=None, callbacks: list | None = None,
                 compute_loss: Callable | None = None, compute_metrics: Callable | None = None,
                 train_dataset=None, eval_dataset=None, data_collator: Callable | None = None, *,
                 optimizers: tuple | None = None, loss_fn: Callable | None = None):
        """`optimizers` = (optimizer, scheduler) and `loss_fn(outputs_or_logits, labels)` are the reference's spellings
        (data_pipeline/trainer/base.py:150-190) of `optimizer` / `scheduler` and of a loss computed from the model's
        output and the batch's labels."""
        if optimizers is not None:
            optimizer = optimizer if optimizer is not None else optimizers[0]
            scheduler = scheduler if scheduler is not None else (optimizers[1] if len(optimizers) > 1 else None)
        if loss_fn is not None and compute_loss is None:
            def compute_loss(m, batch, _f=loss_fn):
                out = m(**{k: v for k, v in batch.items() if k not in ("labels",)})
                out = out.logits if hasattr(out, "logits") else (out[0] if isinstance(out, tuple) else out)
                return _f(out, batch["labels"])
        self.model, self.args = model, args or TrainingArguments()
        self.train_dataset, self.eval_dataset, self.data_collator = train_dataset, eval_dataset, data_collator
        if train_dataloader is None and train_dataset is not None:
            train_dataloader = self.get_train_dataloader()
        if eval_dataloader is None and eval_dataset is not None:
            eval_dataloader = self.get_eval_dataloader()
        self.train_dataloader, self.eval_dataloader = train_dataloader, eval_dataloader
        self.optimizer, self.scheduler = optimizer, scheduler
        self.callbacks = CallbackHandler(callbacks or [])
        self.compute_loss_fn, self.compute_metrics = compute_loss, compute_metrics
        self.state = _State()
        self.device = next(model.parameters()).device
        self.ctx = CallbackContext(trainer=self, state=self.state, config=self.args, model=model)
        self.callbacks.fire("on_init_end", self.ctx)

    def _loader(self, dataset, batch_size: int, shuffle: bool, drop_last: bool):
        from torch.utils.data import DataLoader
        a = self.args
        g = torch.Generator().manual_seed(a.seed) if shuffle else None
        return DataLoader(dataset, batch_size=batch_size, shuffle=shuffle, num_workers=a.dataloader_num_workers,
                          pin_memory=a.dataloader_pin_memory and torch.cuda.is_available(), drop_last=drop_last,
                          collate_fn=self.data_collator, generator=g)

    def get_train_dataloader(self):
        """Shuffled loader over `train_dataset` (data_pipeline/trainer/base.py:333-345); the shuffle is seeded by
        `args.seed`."""
        if self.train_dataset is None:
            from ..core.errors import ConfigurationError
            raise ConfigurationError("training dataset not provided")
        return self._loader(self.train_dataset, self.args.per_device_train_batch_size, True, self.args.dataloader_drop_last)

    def get_eval_dataloader(self):
        if self.eval_dataset is None:
            from ..core.errors import ConfigurationError
            raise ConfigurationError("evaluation dataset not provided")
        return self._loader(self.eval_dataset, self.args.per_device_eval_batch_size or self.args.per_device_train_batch_size,
                            False, False)

    def create_optimizer(self):
        a = self.args
        return create_optimizer(list(self.model.parameters()), name="adamw" if a.optim.startswith("adam") else a.optim,
                                lr=a.learning_rate, weight_decay=a.weight_decay)

    def compute_loss(self, batch: dict) -> torch.Tensor:
        if self.compute_loss_fn is not None:
            return self.compute_loss_fn(self.model, batch)
        out = self.model(**{k: v for k, v in batch.items() if k in ("input_ids", "attention_mask", "labels")})
        return out.loss if hasattr(out, "loss") else out[0]

    def _to_device(self, batch):
        return {k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in batch.items()}

    def train(self, resume_from_checkpoint: str | None = None) -> dict:
        """`resume_from_checkpoint`: a folder written by `save_model`; its weights are loaded before the loop."""
        if resume_from_checkpoint:
            self.load_model(resume_from_checkpoint)
        a = self.args
        if self.optimizer is None:
            self.optimizer = self.create_optimizer()
        steps_per_epoch = max(1, len(self.train_dataloader) // a.gradient_accumulation_steps)
        total = a.max_steps if a.max_steps > 0 else int(steps_per_epoch * a.num_train_epochs)
        self.state.max_steps = total
        if self.scheduler is None:
            self.scheduler = create_scheduler(self.optimizer, a.lr_scheduler_type, total, a.warmup_steps, a.warmup_ratio)
        self.callbacks.fire("on_train_begin", self.ctx)
        self.model.train()
        losses = []
        done = False
        for epoch in range(max(1, math.ceil(a.num_train_epochs))):
            self.state.epoch = epoch
            self.callbacks.fire("on_epoch_begin", self.ctx)
            done = self._train_epoch(losses, total)
            self.callbacks.fire("on_epoch_end", self.ctx)
            if a.eval_strategy == "epoch" and self.eval_dataloader is not None:
                self.evaluate()
            if done or self.ctx.should_stop:
                break
        self.callbacks.fire("on_train_end", self.ctx)
        return {"global_step": self.state.global_step, "train_loss": sum(losses) / max(len(losses), 1)}

    def _train_epoch(self, losses: list, total: int) -> bool:
        a = self.args
        for i, batch in enumerate(self.train_dataloader):
            if i % a.gradient_accumulation_steps == 0:
                self.callbacks.fire("on_step_begin", self.ctx)
            loss = self.compute_loss(self._to_device(batch)) / a.gradient_accumulation_steps
            loss.backward()
            if (i + 1) % a.gradient_accumulation_steps:
                continue
            if a.max_grad_norm and a.max_grad_norm > 0:
                clip_grad_norm_(self.model.parameters(), a.max_grad_norm)
            self.optimizer.step()
            self.scheduler.step()
            self.optimizer.zero_grad(set_to_none=True)
            self.state.global_step += 1
            losses.append(float(loss.detach()) * a.gradient_accumulation_steps)
            self.after_step()
            self.ctx.logs = {"loss": losses[-1], "lr": self.optimizer.param_groups[0]["lr"]}
            self.ctx.should_log = False
            self.callbacks.fire("on_step_end", self.ctx)
            if self.ctx.should_log or self.state.global_step % max(1, a.logging.logging_steps) == 0:
                self.callbacks.fire("on_log", self.ctx)
            if a.eval_strategy == "steps" and a.eval_steps and self.state.global_step % a.eval_steps == 0 \
                    and self.eval_dataloader is not None:
                self.evaluate()
            if self.state.global_step >= total or self.ctx.should_stop:
                return True
        return False

    def after_step(self):
        pass

    @torch.no_grad()
    def evaluate(self) -> dict:
        self.model.eval()
        tot, n = 0.0, 0
        for batch in self.eval_dataloader:
            tot += float(self.compute_loss(self._to_device(batch)))
            n += 1
            self.callbacks.fire("on_prediction_step", self.ctx)
        self.model.train()
        m = {"eval_loss": tot / max(n, 1)}
        if self.compute_metrics is not None:
            m.update(self.compute_metrics(m) or {})
        self.ctx.metrics = m
        self.callbacks.fire("on_evaluate", self.ctx)
        return m

    @torch.no_grad()
    def predict(self, dataloader: Iterable = None, *, dataset=None) -> list:
        """Model outputs per batch.  `dataset=` (a map-style dataset) is batched with the evaluation settings."""
        if dataset is not None:
            dataloader = self._loader(dataset, self.args.per_device_eval_batch_size or self.args.per_device_train_batch_size,
                                      False, False)
        self.model.eval()
        outs = []
        for batch in dataloader:
            out = self.model(**{k: v for k, v in self._to_device(batch).items() if k in ("input_ids", "attention_mask")})
            outs.append(out.logits if hasattr(out, "logits") else out)
        return outs

    def save_model(self, output_dir: str):
        from ..ckpt import save_model_weights
        from pathlib import Path
        save_model_weights(self.model, Path(output_dir))
        self.callbacks.fire("on_save", self.ctx)

    def load_model(self, checkpoint_dir: str) -> None:
        """Weights written by `save_model` (safetensors, sharded or not), or a plain `model.pt` state dict."""
        from pathlib import Path
        d = Path(checkpoint_dir)
        if (d / "model.pt").exists() and not any(d.glob("*.safetensors")):
            self.model.load_state_dict(torch.load(d / "model.pt", map_location=self.device, weights_only=True))
            return
        from ..ckpt import load_model_weights
        load_model_weights(self.model, d)


class PretrainingTrainer(Trainer):
    """Adds an EMA copy of the weights and a curriculum on the sequence length."""

    def __init__(self, *a, ema_decay: float | None = None, curriculum: tuple[int, int, int] | None = None, **kw):
        super().__init__(*a, **kw)
        self.ema_decay = ema_decay
        self.ema = copy.deepcopy(self.model).eval() if ema_decay else None
        self.curriculum = curriculum   # (start_len, end_len, ramp_steps)

    @property
    def ema_model(self):
        """The exponential-moving-average copy of the weights (None when `ema_decay` is not set)."""
        return self.ema

    def current_seq_len(self) -> int | None:
        if not self.curriculum:
            return None
        s, e, ramp = self.curriculum
        return int(s + (e - s) * min(1.0, self.state.global_step / max(1, ramp)))

    def compute_loss(self, batch):
        n = self.current_seq_len()
        if n is not None:
            batch = {k: (v[:, :n] if torch.is_tensor(v) and v.dim() == 2 else v) for k, v in batch.items()}
        return super().compute_loss(batch)

    @torch.no_grad()
    def after_step(self):
        if self.ema is not None:
            for p, q in zip(self.ema.parameters(), self.model.parameters()):
                p.lerp_(q.detach(), 1 - self.ema_decay)


class FineTuningTrainer(Trainer):
    """Layer-wise learning-rate decay: layer l of L gets lr * decay^(L - l)."""

    def __init__(self, *a, layerwise_lr_decay: float | None = None, **kw):
        self.layerwise_lr_decay = layerwise_lr_decay
        super().__init__(*a, **kw)

    def create_optimizer(self):
        if not self.layerwise_lr_decay:
            return super().create_optimizer()
        layers = getattr(getattr(self.model, "model", self.model), "layers", None)
        L = len(layers) if layers is not None else 0
        groups, seen = [], set()
        for l in range(L):
            ps = list(layers[l].parameters())
            seen.update(id(p) for p in ps)
            groups.append({"params": ps, "lr": self.args.learning_rate * self.layerwise_lr_decay ** (L - l)})
        rest = [p for p in self.model.parameters() if id(p) not in seen]
        groups.append({"params": rest, "lr": self.args.learning_rate})
        from ..optim import AdamW
        return AdamW(groups, lr=self.args.learning_rate, weight_decay=self.args.weight_decay)


class Seq2SeqTrainer(Trainer):
    def __init__(self, *a, teacher_forcing_ratio: float = 1.0, scheduled_sampling: bool = False, num_beams: int = 1,
                 length_penalty: float = 1.0, **kw):
        """`num_beams` / `length_penalty` are handed to the model's own `generate`; `teacher_forcing_ratio` < 1 (or
        `scheduled_sampling`, which decays the ratio linearly over training) replaces that fraction of the decoder inputs
        by the model's own greedy predictions from a first, gradient-free pass."""
        super().__init__(*a, **kw)
        self.teacher_forcing_ratio, self.scheduled_sampling = float(teacher_forcing_ratio), scheduled_sampling
        self.num_beams, self.length_penalty = num_beams, length_penalty

    def _decoder_inputs(self, batch):
        ratio = self.teacher_forcing_ratio
        if self.scheduled_sampling and self.state.max_steps:
            ratio = max(0.0, 1.0 - self.state.global_step / self.state.max_steps)
        if ratio >= 1.0 or "decoder_input_ids" not in batch or not self.model.training:
            return batch
        with torch.no_grad():
            out = self.model(**{k: v for k, v in batch.items() if k in ("input_ids", "attention_mask", "decoder_input_ids")})
            logits = out.logits if hasattr(out, "logits") else (out[0] if isinstance(out, tuple) else out)
            own = logits.argmax(-1)
        dec = batch["decoder_input_ids"]
        shifted = torch.cat((dec[:, :1], own[:, :-1]), 1)               # prediction for position t feeds position t+1
        use_own = torch.rand(dec.shape, device=dec.device) >= ratio
        use_own[:, 0] = False
        return {**batch, "decoder_input_ids": torch.where(use_own, shifted, dec)}

    def compute_loss(self, batch):
        batch = self._decoder_inputs(batch)
        out = self.model(**{k: v for k, v in batch.items() if k in ("input_ids", "attention_mask", "decoder_input_ids", "labels")})
        if hasattr(out, "loss") and out.loss is not None:
            return out.loss
        logits = out.logits if hasattr(out, "logits") else out
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), batch["labels"].reshape(-1), ignore_index=-100)

    @torch.no_grad()
    def generate(self, inputs: dict, max_length: int = 128, num_beams: int | None = None,
                 decoder_start_token_id: int = 1, eos_token_id: int | None = None) -> torch.Tensor:
        """Decoder ids for an encoder-decoder model: the model's own `generate` when it has one (beam search and the
        rest), else greedy decoding that feeds `decoder_input_ids` back (data_pipeline/trainer/trainers/__init__.py:242)."""
        self.model.eval()
        inputs = self._to_device(inputs)
        if hasattr(self.model, "generate"):
            kw = {"num_beams": num_beams} if num_beams else {}
            return self.model.generate(**inputs, max_length=max_length, **kw)
        B = inputs["input_ids"].shape[0]
        dec = torch.full((B, 1), decoder_start_token_id, dtype=torch.long, device=self.device)
        done = torch.zeros(B, dtype=torch.bool, device=self.device)
        for _ in range(max_length - 1):
            out = self.model(**inputs, decoder_input_ids=dec)
            logits = out.logits if hasattr(out, "logits") else out[0] if isinstance(out, tuple) else out
            nxt = logits[:, -1].argmax(-1)
            if eos_token_id is not None:
                nxt = torch.where(done, torch.full_like(nxt, eos_token_id), nxt)
                done |= nxt == eos_token_id
            dec = torch.cat((dec, nxt[:, None]), 1)
            if eos_token_id is not None and bool(done.all()):
                break
        return dec


class TextGenerationTrainer(Trainer):
    def __init__(self, *a, top_k: int = 0, top_p: float = 1.0, temperature: float = 1.0, repetition_penalty: float = 1.0,
                 **kw):
        """Sampling defaults of `generate` (each call may override them)."""
        super().__init__(*a, **kw)
        self.top_k, self.top_p, self.temperature, self.repetition_penalty = top_k, top_p, temperature, repetition_penalty

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32, temperature: float | None = None,
                 top_k: int | None = None, top_p: float | None = None, eos_token_id: int | None = None,
                 do_sample: bool = True) -> torch.Tensor:
        """`do_sample=False`: greedy decoding (temperature 0)."""
        from ..inference.sampling import sample
        temperature = self.temperature if temperature is None else temperature
        top_k = self.top_k if top_k is None else top_k
        top_p = self.top_p if top_p is None else top_p
        if not do_sample:
            temperature = 0.0
        self.model.eval()
        ids = input_ids.to(self.device)
        for _ in range(max_new_tokens):
            out = self.model(input_ids=ids)
            logits = (out.logits if hasattr(out, "logits") else out)[:, -1].float()
            B = logits.shape[0]
            if self.repetition_penalty != 1.0:
                seen = torch.zeros_like(logits, dtype=torch.bool).scatter_(1, ids, True)
                logits = torch.where(seen, torch.where(logits > 0, logits / self.repetition_penalty,
                                                       logits * self.repetition_penalty), logits)
            nxt, _ = sample(logits, [temperature] * B, [top_k] * B, [top_p] * B, [0.0] * B, [None] * B)
            ids = torch.cat((ids, nxt.unsqueeze(1)), dim=1)
            if eos_token_id is not None and bool((nxt == eos_token_id).all()):
                break
        return ids


@dataclass
class TrainOutput:
    """What a training run produced (data_pipeline/trainer/base.py:103)."""
    global_step: int
    training_loss: float
    metrics: dict = field(default_factory=dict)

    def __repr__(self) -> str:
        return f"TrainOutput(global_step={self.global_step}, training_loss={self.training_loss:.6f}, metrics={self.metrics})"

    @classmethod
    def from_summary(cls, summary: dict) -> "TrainOutput":
        """From the dictionary `Trainer.train()` returns."""
        loss = summary.get("train_loss", summary.get("training_loss", float("nan")))
        return cls(int(summary.get("global_step", 0)), float(loss),
                   {k: v for k, v in summary.items() if k not in ("global_step",)})


@dataclass
class PredictionOutput:
    predictions: torch.Tensor
    label_ids: torch.Tensor | None = None
    metrics: dict = field(default_factory=dict)


# ---- type aliases of data_pipeline/trainer/base.py
BatchType = dict[str, torch.Tensor]
MetricsType = dict[str, float]
