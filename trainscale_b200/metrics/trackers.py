"""Training-time trackers: loss, next-token accuracy, gradient health and their bundle.

Method surface of data_pipeline/trainer/metrics/loss.py:32-420 (`LossTracker`, `AccuracyTracker`), gradient.py:30-350
(`GradientTracker`) and training.py:35-335 (`TrainingMetrics`).  What differs from the reference: statistics that come
from tensors are reduced ON THE DEVICE and read with a single host transfer per update (the reference calls `.item()`
several times per parameter), and `update()` also accepts an already computed norm / loss, which is what this
framework's engines hand over (they form the gradient norm inside the fused reduce-scatter kernel).
"""
from __future__ import annotations

import math
from collections import deque
from typing import Iterable

import torch

from ..utils.refargs import ANY, reference_kwargs
import torch.distributed as dist

from .throughput import ThroughputTracker

_HISTORY = 1000


def _all_reduce_sum(values: list[float], group=None) -> list[float]:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return values
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    dist.all_reduce(t, group=group)
    return t.tolist()


class LossTracker:
    """Token-weighted running loss, exponential moving average, perplexity, bounded history."""

    def __init__(self, ema_decay: float = 0.99, window: int = 100):
        self.ema_decay = self.decay = ema_decay
        self.window = deque(maxlen=window)
        self.reset()

    def reset(self) -> None:
        self.sum, self.tokens, self.samples, self.steps = 0.0, 0, 0, 0
        self.ema, self._last = None, 0.0
        self._history: list[float] = []
        self.window.clear()

    def update(self, loss, num_tokens: int = 1, num_samples: int = 1, accumulation_steps: int = 1) -> None:
        """`loss` is the mean over `num_tokens`; pass `accumulation_steps` if it was already divided by them."""
        l = float(loss.detach()) if torch.is_tensor(loss) else float(loss)
        l *= accumulation_steps
        if not math.isfinite(l):
            return
        self.ema = l if self.ema is None else self.ema_decay * self.ema + (1 - self.ema_decay) * l
        self.sum += l * num_tokens
        self.tokens += num_tokens
        self.samples += num_samples
        self.steps += 1
        self._last = l
        self.window.append(l)
        if len(self._history) < _HISTORY:
            self._history.append(l)

    def update_from_logits(self, logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> float:
        """Cross-entropy of [B, T, V] logits against [B, T] labels with the causal shift ([N, V] / [N]: no shift)."""
        if logits.dim() == 3:
            logits, labels = logits[..., :-1, :], labels[..., 1:]
        z, y = logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1)
        both = torch.stack((torch.nn.functional.cross_entropy(z, y, ignore_index=ignore_index, reduction="sum"),
                            (y != ignore_index).sum().float())).tolist()             # one host read
        if both[1] == 0:
            return 0.0
        self.update(both[0] / both[1], num_tokens=int(both[1]), num_samples=logits.shape[0] if logits.dim() == 3 else 1)
        return both[0] / both[1]

    # the reference's accessor names
    def compute_avg(self) -> float: return self.sum / self.tokens if self.tokens else 0.0
    def compute_ema(self) -> float: return self.ema if self.ema is not None else 0.0
    def compute_ppl(self) -> float: return math.exp(min(self.compute_avg(), 50.0))
    def compute_ppl_ema(self) -> float: return math.exp(min(self.compute_ema(), 50.0))

    def compute_variance(self) -> float:
        h = self._history
        if len(h) < 2:
            return 0.0
        m = sum(h) / len(h)
        return sum((x - m) ** 2 for x in h) / (len(h) - 1)

    def get_history(self, last_n: int | None = None) -> list[float]:
        return list(self._history if last_n is None else self._history[-last_n:])

    last_loss = property(lambda self: self._last)
    total_tokens = property(lambda self: self.tokens)
    total_samples = property(lambda self: self.samples)
    step_count = property(lambda self: self.steps)
    # this framework's shorter names
    mean = property(lambda self: self.sum / max(self.tokens, 1))
    perplexity = property(lambda self: math.exp(min(self.mean, 50.0)))
    windowed = property(lambda self: sum(self.window) / max(len(self.window), 1))

    def sync(self, process_group=None) -> float:
        """Sum the running totals over the ranks (in place); returns the global token-weighted mean."""
        self.sum, tokens, samples = _all_reduce_sum([self.sum, float(self.tokens), float(self.samples)], process_group)
        self.tokens, self.samples = int(tokens), int(samples)
        return self.compute_avg()

    def state_dict(self) -> dict:
        return {"ema": self.ema, "sum": self.sum, "tokens": self.tokens, "samples": self.samples, "steps": self.steps,
                "last": self._last, "history": list(self._history[-100:])}

    @reference_kwargs(state="sd")
    def load_state_dict(self, sd: dict) -> None:
        self.ema, self.sum, self.tokens = sd.get("ema"), sd.get("sum", 0.0), sd.get("tokens", 0)
        self.samples, self.steps, self._last = sd.get("samples", 0), sd.get("steps", 0), sd.get("last", 0.0)
        self._history = list(sd.get("history", []))


class AccuracyTracker:
    """Next-token accuracy with the causal shift (logits[..., :-1] against labels[..., 1:])."""

    def __init__(self, ignore_index: int = -100):
        self.ignore_index = ignore_index
        self.reset()

    def reset(self) -> None:
        self.correct, self.total = 0, 0

    def update(self, correct: int, total: int) -> None:
        self.correct += int(correct)
        self.total += int(total)

    def update_from_logits(self, logits: torch.Tensor, labels: torch.Tensor, ignore_index: int | None = None) -> float:
        ig = self.ignore_index if ignore_index is None else ignore_index
        if logits.dim() == 3:
            logits, labels = logits[..., :-1, :], labels[..., 1:]
        p, t = logits.argmax(-1), labels
        m = t != ig
        c, n = torch.stack((((p == t) & m).sum(), m.sum())).tolist()               # one host read
        self.update(c, n)
        return c / n if n else 0.0

    def compute(self) -> float:
        return self.correct / self.total if self.total else 0.0

    accuracy = property(lambda self: self.compute())

    def sync(self, process_group=None) -> float:
        c, n = _all_reduce_sum([float(self.correct), float(self.total)], process_group)
        self.correct, self.total = int(c), int(n)
        return self.compute()


class GradientTracker:
    """Gradient health: global norm, its EMA and history, mean / variance of the gradient values, NaN / Inf flags,
    per-layer norms.  `update(x)` takes parameters (an iterable), a module, or a norm that was computed elsewhere."""

    def __init__(self, max_norm: float = 10.0, ema_decay: float = 0.99, window: int = 100,
                 explode_threshold: float = 1e6):
        self.max_norm, self.ema_decay, self.threshold = max_norm, ema_decay, explode_threshold
        self.norms = deque(maxlen=window)
        self.reset()

    def reset(self) -> None:
        self._norm, self._ema, self._steps = 0.0, None, 0
        self._nan = self._inf = False
        self._count, self._sum, self._sq = 0, 0.0, 0.0
        self._history: list[float] = []
        self._layers: dict[str, float] = {}
        self.nan_count, self.clipped = 0, 0
        self.norms.clear()

    def _record(self, norm: float, max_norm: float | None = None) -> float:
        self._steps += 1
        if not math.isfinite(norm):
            self.nan_count += 1
            self._norm = norm
            return norm
        self._norm = norm
        self._ema = norm if self._ema is None else self.ema_decay * self._ema + (1 - self.ema_decay) * norm
        self.norms.append(norm)
        if len(self._history) < _HISTORY:
            self._history.append(norm)
        if max_norm and norm > max_norm:
            self.clipped += 1
        return norm

    def update(self, parameters, named_parameters=None, max_norm: float | None = None) -> float:
        if isinstance(parameters, (int, float)) or (torch.is_tensor(parameters) and parameters.dim() == 0):
            g = float(parameters)
            self._nan, self._inf = math.isnan(g), math.isinf(g)
            return self._record(g, max_norm)
        if isinstance(parameters, torch.nn.Module):
            named_parameters, parameters = parameters.named_parameters(), None
        items = list(named_parameters) if named_parameters is not None else [(None, p) for p in parameters]
        items = [(n, p.grad.detach()) for n, p in items if p.grad is not None]
        if not items:
            return self._record(0.0, max_norm)
        # [k, 4] statistics on the device: sum of squares, sum, any NaN, any Inf - one transfer for everything
        rows = torch.stack([torch.stack((g.float().pow(2).sum(), g.float().sum(), torch.isnan(g).any().float(),
                                         torch.isinf(g).any().float())) for _, g in items]).tolist()
        sq = sum(r[0] for r in rows)
        self._sq, self._sum = sq, sum(r[1] for r in rows)
        self._nan, self._inf = any(r[2] for r in rows), any(r[3] for r in rows)
        self._count = sum(g.numel() for _, g in items)
        self._layers = {n: math.sqrt(r[0]) for (n, _), r in zip(items, rows) if n is not None}
        return self._record(math.sqrt(sq) if math.isfinite(sq) else float("nan"), max_norm)

    def update_from_model(self, model: torch.nn.Module) -> float:
        return self.update(model)

    def compute_norm(self) -> float: return self._norm
    def compute_ema_norm(self) -> float: return self._ema if self._ema is not None else 0.0
    def compute_mean(self) -> float: return self._sum / self._count if self._count else 0.0

    def compute_variance(self) -> float:
        if not self._count:
            return 0.0
        m = self._sum / self._count
        return max(self._sq / self._count - m * m, 0.0)

    def compute_std(self) -> float: return math.sqrt(self.compute_variance())
    def has_nan(self) -> bool: return bool(self._nan)
    def has_inf(self) -> bool: return bool(self._inf)
    def has_nan_or_inf(self) -> bool: return bool(self._nan or self._inf)
    def is_anomaly(self) -> bool: return self.has_nan_or_inf() or not math.isfinite(self._norm) or self._norm > self.max_norm
    def exploding(self) -> bool: return bool(self.norms) and self.norms[-1] > self.threshold
    def get_layer_norms(self) -> dict: return dict(self._layers)

    def get_top_layers(self, k: int = 5) -> list:
        return sorted(self._layers.items(), key=lambda kv: kv[1], reverse=True)[:k]

    def histogram(self) -> dict:
        h = sorted(self._history)
        if not h:
            return {"p10": 0, "p25": 0, "p50": 0, "p75": 0, "p90": 0, "max": 0}
        pick = lambda p: h[min(int(p * len(h) / 100), len(h) - 1)]      # noqa: E731
        return {"p10": pick(10), "p25": pick(25), "p50": pick(50), "p75": pick(75), "p90": pick(90), "max": h[-1]}

    step_count = property(lambda self: self._steps)
    mean = property(lambda self: sum(self.norms) / max(len(self.norms), 1))

    def log_dict(self) -> dict:
        return {"gradient/norm": self._norm, "gradient/norm_ema": self.compute_ema_norm(),
                "gradient/mean": self.compute_mean(), "gradient/std": self.compute_std(),
                "gradient/has_nan": float(self._nan), "gradient/has_inf": float(self._inf)}

    def state_dict(self) -> dict:
        return {"norms": list(self.norms), "nan_count": self.nan_count, "clipped": self.clipped, "ema": self._ema,
                "steps": self._steps, "history": list(self._history[-100:])}

    @reference_kwargs(state="sd")
    def load_state_dict(self, sd: dict) -> None:
        self.norms.extend(sd.get("norms", []))
        self.nan_count, self.clipped = sd.get("nan_count", 0), sd.get("clipped", 0)
        self._ema, self._steps, self._history = sd.get("ema"), sd.get("steps", 0), list(sd.get("history", []))


class TrainingMetrics:
    """The trackers a training loop feeds, behind one `update_step(...)`, with step / epoch counters, reduction over
    the ranks, a flat dictionary for loggers and a one-line summary."""

    def __init__(self, flops_per_token: float = 0.0, world_size: int = 1, distributed: bool = False,
                 log_prefix: str = "train", model_params: int | None = None):
        self.distributed, self.log_prefix, self.model_params = distributed, log_prefix, model_params
        if model_params and not flops_per_token:
            flops_per_token = 6.0 * model_params
        self.loss, self.accuracy, self.gradient = LossTracker(), AccuracyTracker(), GradientTracker()
        self.throughput = ThroughputTracker(flops_per_token, world_size=world_size)
        self._lr, self._global_step, self._epoch, self._epoch_step = 0.0, 0, 0, 0

    acc = property(lambda self: self.accuracy)
    grad = property(lambda self: self.gradient)

    def reset(self) -> None:
        """Start a new accumulation interval (the counters of the run and the throughput clock keep going)."""
        self.loss.reset()
        self.accuracy.reset()

    def reset_all(self) -> None:
        self.reset()
        self.gradient.reset()
        self.throughput.reset()
        self._global_step = self._epoch = self._epoch_step = 0

    def start(self) -> None:
        self.throughput.start()

    def new_epoch(self, epoch: int) -> None:
        self._epoch, self._epoch_step = epoch, 0

    def update_step(self, loss, logits=None, labels=None, model=None, parameters=None, batch_size: int = 1,
                    num_tokens: int = 0, lr: float | None = None, grad_norm: float | None = None,
                    accumulation_steps: int = 1) -> None:
        self.loss.update(loss, max(num_tokens, 1), batch_size, accumulation_steps)
        if logits is not None and labels is not None:
            self.accuracy.update_from_logits(logits, labels)
        self.throughput.update(samples=batch_size, tokens=num_tokens)
        if grad_norm is not None:
            self.gradient.update(grad_norm)
        elif model is not None:
            self.gradient.update(model)
        elif parameters is not None:
            self.gradient.update(parameters)
        if lr is not None:
            self._lr = lr
        self._global_step += 1
        self._epoch_step += 1

    def sync(self, process_group=None) -> None:
        if self.distributed:
            self.loss.sync(process_group)
            self.accuracy.sync(process_group)
            self.throughput.sync(process_group)

    def compute(self, sync: bool = True) -> dict:
        if sync:
            self.sync()
        t = self.throughput
        return {"loss": self.loss.compute_avg(), "loss_ema": self.loss.compute_ema(), "ppl": self.loss.compute_ppl(),
                "accuracy": self.accuracy.compute(), "tokens_per_sec": t.tokens_per_sec(),
                "samples_per_sec": t.samples_per_sec(), "grad_norm": self.gradient.compute_norm(),
                "grad_norm_ema": self.gradient.compute_ema_norm(), "mfu": t.compute_mfu(), "lr": self._lr,
                "global_step": self._global_step, "epoch": self._epoch, "epoch_step": self._epoch_step,
                "total_tokens": t.total_tokens, "elapsed_seconds": t.elapsed_seconds()}

    def log_dict(self, sync: bool = True) -> dict:
        m = self.compute(sync)
        pre = f"{self.log_prefix}/" if self.log_prefix else ""
        out = {f"{pre}{k}": m[k] for k in ("loss", "loss_ema", "ppl", "accuracy", "tokens_per_sec", "samples_per_sec",
                                            "grad_norm", "mfu", "lr")}
        out[f"{pre}step"] = float(m["global_step"])
        return out

    def format_log_string(self, sync: bool = True) -> str:
        m = self.compute(sync)
        ppl = f"ppl={m['ppl']:.2e}" if m["ppl"] > 1000 else f"ppl={m['ppl']:.2f}"
        parts = [f"step={m['global_step']}", f"loss={m['loss']:.4f}", ppl, f"acc={m['accuracy']:.2%}",
                 f"tok/s={m['tokens_per_sec']:,.0f}", f"grad={m['grad_norm']:.3f}", f"lr={m['lr']:.2e}"]
        if m["mfu"] > 0:
            parts.append(f"mfu={m['mfu']:.1%}")
        return " | ".join(parts)

    def summary(self) -> dict:
        return {"loss": self.loss.mean, "loss_ema": self.loss.ema, "ppl": self.loss.perplexity,
                "acc": self.accuracy.accuracy, "grad_norm": self.gradient.mean,
                "tokens_per_second": self.throughput.tokens_per_second(), "mfu": self.throughput.compute_mfu()}

    def state_dict(self) -> dict:
        return {"loss": self.loss.state_dict(), "grad": self.gradient.state_dict(),
                "throughput": self.throughput.state_dict(), "lr": self._lr, "global_step": self._global_step,
                "epoch": self._epoch, "epoch_step": self._epoch_step}

    @reference_kwargs(state="sd")
    def load_state_dict(self, sd: dict) -> None:
        self.loss.load_state_dict(sd.get("loss", {}))
        self.gradient.load_state_dict(sd.get("grad", {}))
        self.throughput.load_state_dict(sd.get("throughput", {"total_tokens": 0, "total_seconds": 0.0}))
        self._lr, self._global_step = sd.get("lr", 0.0), sd.get("global_step", 0)
        self._epoch, self._epoch_step = sd.get("epoch", 0), sd.get("epoch_step", 0)
