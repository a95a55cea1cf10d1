"""Evaluation metrics, training trackers and their distributed reduction.

After data_pipeline/trainer/metrics/*.py: `Metric` ABC with Accuracy / Precision / Recall / F1 / AUROC / Perplexity /
BLEU / ROUGE / MSE / MAE / R2 (`__init__.py:16-433`), `sync_metric(s)` and `DistributedMetricBuffer`
(`distributed.py:53-173`), `GradientTracker` (`gradient.py:30`), `LossTracker` / `AccuracyTracker` (`loss.py:32,309`),
`ThroughputTracker` (`throughput.py:96`), `TrainingMetrics` (`training.py:35`).
"""
from __future__ import annotations

import math
from collections import Counter, deque
from typing import Sequence

import torch
import torch.distributed as dist

from ..utils.refargs import ANY, reference_kwargs

from .throughput import PEAK_TFLOPS, ThroughputTracker, device_peak_tflops  # noqa: F401


@reference_kwargs(operation="op", process_group="group")
def sync_metric(value: float | torch.Tensor, op: str = "mean", group=None) -> float:
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
        return float(value)
    t = torch.as_tensor(float(value), dtype=torch.float64)
    if dist.get_backend(group) == "nccl":
        t = t.float().cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=group)
    return float(t / dist.get_world_size(group)) if op == "mean" else float(t)


@reference_kwargs(metrics="values", operation="op", process_group="group")
def sync_metrics(values: dict[str, float], op: str = "mean", group=None) -> dict[str, float]:
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
        return dict(values)
    keys = sorted(values)
    t = torch.tensor([float(values[k]) for k in keys], dtype=torch.float32)
    if dist.get_backend(group) == "nccl":
        t = t.cuda()
    dist.all_reduce(t, group=group)
    if op == "mean":
        t /= dist.get_world_size(group)
    return dict(zip(keys, t.tolist()))


class DistributedMetricBuffer:
    """Accumulate named sums locally; one all-reduce when read."""

    def __init__(self, operation: str = "mean"):
        if operation not in ("mean", "sum"):
            raise ValueError("operation must be 'mean' or 'sum'")
        self.operation = operation
        self.sums: dict[str, float] = {}
        self._counts: dict[str, int] = {}

    def add(self, name: str, value, weight: float = 1.0):
        if torch.is_tensor(value):
            value = value.detach().item()
        self.sums[name] = self.sums.get(name, 0.0) + float(value) * weight
        self.sums[name + "/weight"] = self.sums.get(name + "/weight", 0.0) + weight
        self._counts[name] = self._counts.get(name, 0) + 1

    # ---- data_pipeline/trainer/metrics/distributed.py:205-255
    def counts(self) -> dict[str, int]:
        return dict(self._counts)

    def local_sums(self) -> dict[str, float]:
        return {k: v for k, v in self.sums.items() if not k.endswith("/weight")}

    def local_means(self) -> dict[str, float]:
        return {k: v / max(self.sums[k + "/weight"], 1e-12) for k, v in self.local_sums().items()}

    def reduce_all(self, process_group=None) -> dict[str, float]:
        """One all-reduce for every buffered name.  'mean' is the mean over ALL values of all ranks (weighted by how
        many each rank added), not the mean of the ranks' means; 'sum' the total."""
        if self.operation == "mean":
            return self.compute(process_group)
        return sync_metrics(self.local_sums(), "sum", process_group)

    def compute(self, group=None) -> dict[str, float]:
        tot = sync_metrics(self.sums, "sum", group)
        return {k: v / max(tot.get(k + "/weight", 1.0), 1e-12) for k, v in tot.items() if not k.endswith("/weight")}

    def reset(self):
        self.sums.clear()
        self._counts.clear()

    clear = reset


def _with_name(init):
    """Constructor wrapper: every metric takes `name=` (the key under which a collection reports it)."""
    import functools
    import inspect

    @functools.wraps(init)
    def wrapper(self, *args, name: str | None = None, **kwargs):
        init(self, *args, **kwargs)
        if name is not None:
            self.name = name
    sig = inspect.signature(init)
    params = list(sig.parameters.values())
    tail = [p for p in params if p.kind is inspect.Parameter.VAR_KEYWORD]
    head = [p for p in params if p.kind is not inspect.Parameter.VAR_KEYWORD]
    if "name" not in sig.parameters:
        head.append(inspect.Parameter("name", inspect.Parameter.KEYWORD_ONLY, default=None))
    wrapper.__signature__ = sig.replace(parameters=head + tail)
    return wrapper


def _with_reference_update(update):
    """`update(predictions=, targets=)`: the reference's names for the first two arguments of any metric's update."""
    import inspect
    names = [p for p in inspect.signature(update).parameters if p != "self"][:2]
    renames = {ref: ours for ref, ours in zip(("predictions", "targets"), names) if ref != ours}
    return reference_kwargs(**renames)(update) if renames else update


class Metric:
    """update / compute / reset; calling a metric resets it, feeds one batch and returns the value
    (data_pipeline/trainer/metrics/__init__.py:16-40).  `name` is the key under which a collection reports it; every
    subclass's constructor takes it as a keyword, and every `update` also answers to `predictions=` / `targets=`."""
    name: str = ""

    def __init__(self, name: str | None = None):
        if name is not None:
            self.name = name

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        if "__init__" in cls.__dict__:
            cls.__init__ = _with_name(cls.__dict__["__init__"])
        if "update" in cls.__dict__:
            cls.update = _with_reference_update(cls.__dict__["update"])

    @reference_kwargs(predictions="preds")
    def update(self, preds, targets): raise NotImplementedError
    def compute(self) -> float: raise NotImplementedError
    def reset(self): raise NotImplementedError

    def __call__(self, preds, targets):
        self.reset()
        self.update(preds, targets)
        return self.compute()

    def named(self, name: str) -> "Metric":
        self.name = name
        return self


class _Counts(Metric):
    def __init__(self, num_classes: int | None = None, average: str = "macro", ignore_index: int = -100, top_k: int = 1):
        self.num_classes, self.average, self.ignore_index, self.top_k = num_classes, average, ignore_index, int(top_k)
        self.reset()

    def reset(self):
        self.tp, self.fp, self.fn, self.correct, self.total = Counter(), Counter(), Counter(), 0, 0

    def update(self, preds, targets):
        p = torch.as_tensor(preds)
        t = torch.as_tensor(targets)
        hits = None
        if p.dim() > t.dim():
            if self.top_k > 1:                      # a hit when the target is among the k highest scores
                topk = p.topk(min(self.top_k, p.shape[-1]), dim=-1).indices.reshape(-1, min(self.top_k, p.shape[-1]))
                hits = (topk == t.reshape(-1, 1)).any(-1)
            p = p.argmax(-1)
        p, t = p.reshape(-1), t.reshape(-1)
        keep = t != self.ignore_index
        p, t = p[keep], t[keep]
        self.correct += int(hits[keep].sum()) if hits is not None else int((p == t).sum())
        self.total += int(t.numel())
        for c in torch.unique(torch.cat((p, t))).tolist():
            self.tp[c] += int(((p == c) & (t == c)).sum())
            self.fp[c] += int(((p == c) & (t != c)).sum())
            self.fn[c] += int(((p != c) & (t == c)).sum())

    def _prf(self):
        classes = sorted(set(self.tp) | set(self.fp) | set(self.fn))
        if self.average == "micro":
            tp, fp, fn = sum(self.tp.values()), sum(self.fp.values()), sum(self.fn.values())
            p = tp / max(tp + fp, 1)
            r = tp / max(tp + fn, 1)
            return p, r, 2 * p * r / max(p + r, 1e-12)
        ps, rs, fs = [], [], []
        for c in classes:
            p = self.tp[c] / max(self.tp[c] + self.fp[c], 1)
            r = self.tp[c] / max(self.tp[c] + self.fn[c], 1)
            ps.append(p)
            rs.append(r)
            fs.append(2 * p * r / max(p + r, 1e-12))
        n = max(len(classes), 1)
        return sum(ps) / n, sum(rs) / n, sum(fs) / n


class Accuracy(_Counts):
    def compute(self): return self.correct / max(self.total, 1)


class Precision(_Counts):
    def compute(self): return self._prf()[0]


class Recall(_Counts):
    def compute(self): return self._prf()[1]


class F1Score(_Counts):
    def compute(self): return self._prf()[2]


class AUROC(Metric):
    def __init__(self): self.reset()
    def reset(self): self.scores, self.labels = [], []

    def update(self, preds, targets):
        self.scores += torch.as_tensor(preds).reshape(-1).tolist()
        self.labels += torch.as_tensor(targets).reshape(-1).tolist()

    def compute(self):
        pairs = sorted(zip(self.scores, self.labels))
        pos = sum(1 for _, l in pairs if l == 1)
        neg = len(pairs) - pos
        if pos == 0 or neg == 0:
            return float("nan")
        rank_sum, i = 0.0, 0
        while i < len(pairs):
            j = i
            while j < len(pairs) and pairs[j][0] == pairs[i][0]:
                j += 1
            avg_rank = (i + j + 1) / 2
            rank_sum += avg_rank * sum(1 for k in range(i, j) if pairs[k][1] == 1)
            i = j
        return (rank_sum - pos * (pos + 1) / 2) / (pos * neg)


class Perplexity(Metric):
    def __init__(self, ignore_index: int = -100):
        self.ignore_index = ignore_index
        self.reset()

    def reset(self): self.nll, self.n = 0.0, 0

    def update(self, logits, targets):
        lp = torch.log_softmax(torch.as_tensor(logits).float(), -1)
        t = torch.as_tensor(targets)
        m = t != self.ignore_index
        self.nll += float(-(lp.gather(-1, t.clamp(min=0).unsqueeze(-1)).squeeze(-1) * m).sum())
        self.n += int(m.sum())

    def update_from_loss(self, mean_loss: float, num_tokens: int):
        self.nll += mean_loss * num_tokens
        self.n += num_tokens

    def compute(self): return math.exp(min(self.nll / max(self.n, 1), 50.0))


def _ngrams(tokens: Sequence, n: int) -> Counter:
    return Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1))


class BLEU(Metric):
    def __init__(self, max_n: int = 4, smooth: bool = True):
        self.max_n, self.smooth = max_n, smooth
        self.reset()

    def reset(self):
        self.match, self.total = [0] * self.max_n, [0] * self.max_n
        self.hyp_len = self.ref_len = 0

    def update(self, hypotheses: Sequence[str | Sequence], references: Sequence[str | Sequence]):
        for h, r in zip(hypotheses, references):
            h = h.split() if isinstance(h, str) else list(h)
            r = r.split() if isinstance(r, str) else list(r)
            self.hyp_len += len(h)
            self.ref_len += len(r)
            for n in range(1, self.max_n + 1):
                hn, rn = _ngrams(h, n), _ngrams(r, n)
                self.match[n - 1] += sum(min(c, rn[g]) for g, c in hn.items())
                self.total[n - 1] += max(len(h) - n + 1, 0)

    def compute(self):
        if self.hyp_len == 0:
            return 0.0
        logs = []
        for m, t in zip(self.match, self.total):
            if self.smooth:
                m, t = m + 1, t + 1
            if m == 0 or t == 0:
                return 0.0
            logs.append(math.log(m / t))
        bp = 1.0 if self.hyp_len > self.ref_len else math.exp(1 - self.ref_len / max(self.hyp_len, 1))
        return bp * math.exp(sum(logs) / self.max_n)


class ROUGE(Metric):
    """ROUGE-1 / ROUGE-2 / ROUGE-L F-measures."""

    def __init__(self): self.reset()
    def reset(self): self.scores = {"rouge1": [], "rouge2": [], "rougeL": []}

    @staticmethod
    def _lcs(a, b):
        dp = [0] * (len(b) + 1)
        for x in a:
            prev = 0
            for j, y in enumerate(b, 1):
                cur = dp[j]
                dp[j] = prev + 1 if x == y else max(dp[j], dp[j - 1])
                prev = cur
        return dp[-1]

    @staticmethod
    def _f(m, h, r):
        if m == 0:
            return 0.0
        p, rc = m / max(h, 1), m / max(r, 1)
        return 2 * p * rc / (p + rc)

    def update(self, hypotheses, references):
        for h, r in zip(hypotheses, references):
            h = h.split() if isinstance(h, str) else list(h)
            r = r.split() if isinstance(r, str) else list(r)
            for n, key in ((1, "rouge1"), (2, "rouge2")):
                hn, rn = _ngrams(h, n), _ngrams(r, n)
                self.scores[key].append(self._f(sum(min(c, rn[g]) for g, c in hn.items()), sum(hn.values()), sum(rn.values())))
            self.scores["rougeL"].append(self._f(self._lcs(h, r), len(h), len(r)))

    def compute(self):
        return {k: sum(v) / max(len(v), 1) for k, v in self.scores.items()}


class _Regression(Metric):
    def __init__(self): self.reset()
    def reset(self): self.p, self.t = [], []

    def update(self, preds, targets):
        self.p.append(torch.as_tensor(preds).float().reshape(-1))
        self.t.append(torch.as_tensor(targets).float().reshape(-1))

    def _cat(self): return torch.cat(self.p), torch.cat(self.t)


class MSE(_Regression):
    def compute(self):
        p, t = self._cat()
        return float(((p - t) ** 2).mean())


class MAE(_Regression):
    def compute(self):
        p, t = self._cat()
        return float((p - t).abs().mean())


class R2Score(_Regression):
    def compute(self):
        p, t = self._cat()
        return float(1 - ((p - t) ** 2).sum() / ((t - t.mean()) ** 2).sum().clamp(min=1e-12))


from .trackers import AccuracyTracker, GradientTracker, LossTracker, TrainingMetrics  # noqa: E402,F401


# ------------------------------------------------------------------------------------------------ names of the reference
for _cls, _name in ((Accuracy, "accuracy"), (Precision, "precision"), (Recall, "recall"), (F1Score, "f1"),
                    (AUROC, "auroc"), (Perplexity, "perplexity"), (BLEU, "bleu"), (ROUGE, "rouge"), (MSE, "mse"),
                    (MAE, "mae"), (R2Score, "r2")):
    _cls.name = _name

BLEUScore = BLEU
MeanSquaredError = MSE
MeanAbsoluteError = MAE


class ROUGEScore(ROUGE):
    """ROUGE-L F-measure as one number (data_pipeline/trainer/metrics/__init__.py:310-343); `ROUGE` reports
    ROUGE-1 / -2 / -L together."""
    name = "rouge_l"

    def compute(self) -> float:
        return super().compute()["rougeL"]


class MetricCollection:
    """Several metrics fed with the same batches; `compute()` returns {metric name: value}
    (data_pipeline/trainer/metrics/__init__.py:415-434)."""

    def __init__(self, metrics: Sequence[Metric] = ()):
        self.metrics: dict[str, Metric] = {}
        for m in metrics:
            self.add(m)

    def add(self, metric: Metric) -> None:
        self.metrics[metric.name or type(metric).__name__.lower()] = metric

    @reference_kwargs(predictions="preds")
    def update(self, preds, targets) -> None:
        for m in self.metrics.values():
            m.update(preds, targets)

    def compute(self) -> dict:
        return {n: m.compute() for n, m in self.metrics.items()}

    def reset(self) -> None:
        for m in self.metrics.values():
            m.reset()


def compute_accuracy(preds, targets) -> float:
    return Accuracy()(preds, targets)


def compute_f1(preds, targets, average: str = "macro") -> float:
    return F1Score(average=average)(preds, targets)


def compute_perplexity(preds, targets) -> float:
    return Perplexity()(preds, targets)


def create_training_metrics(distributed: bool = False, model=None, log_prefix: str = "train") -> TrainingMetrics:
    """`TrainingMetrics` with the model's parameter count turned into FLOPs per token (6 N) for the MFU figure
    (data_pipeline/trainer/metrics/training.py:337-360)."""
    n = sum(p.numel() for p in model.parameters()) if model is not None else 0
    world = dist.get_world_size() if distributed and dist.is_available() and dist.is_initialized() else 1
    return TrainingMetrics(flops_per_token=6.0 * n, world_size=world, distributed=distributed, log_prefix=log_prefix,
                           model_params=n or None)


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size() -> int:
    return dist.get_world_size() if is_distributed() else 1


def get_rank() -> int:
    return dist.get_rank() if is_distributed() else 0


def is_main_process() -> bool:
    return get_rank() == 0
