"""Losses beyond the language-model set: feature / attention distillation, robust regression, perceptual, listwise
ranking, segmentation and detection.  Plain PyTorch math (none of these is on an LLM training step's hot path), written
vectorised: no Python loop over list positions, bins or pairs.

Reference: data_pipeline/trainer/loss/sota_losses.py:72 (LossOutput), :1025-1150 (distillation), :2185-2284
(Charbonnier, perceptual), :2317-2496 (ListMLE, LambdaRank), :2636-2908 (focal Tversky, GHM-C, IoU, boundary), :3183.
"""
from __future__ import annotations

from typing import NamedTuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class LossOutput(NamedTuple):
    """Loss with the metrics to log beside it and an optional auxiliary term (router balance and the like)."""
    loss: torch.Tensor
    metrics: dict
    aux_loss: torch.Tensor | None = None


def _reduce(x: torch.Tensor, reduction: str) -> torch.Tensor:
    if reduction == "mean":
        return x.mean()
    if reduction == "sum":
        return x.sum()
    return x


class FeatureDistillationLoss(nn.Module):
    """Match intermediate representations of a student to a teacher's: `mse`, `l1` or `cosine` distance, optionally
    on L2-normalised features.  When the widths differ a bias-free projection of the student is created on first use
    (to `projection_dim` if given, else to the teacher's width) and trained with the student."""

    def __init__(self, loss_type: str = "mse", normalize: bool = True, projection_dim: int | None = None):
        super().__init__()
        if loss_type not in ("mse", "cosine", "l1"):
            raise ValueError(f"unknown loss_type {loss_type!r}")
        self.loss_type, self.normalize, self.projection_dim = loss_type, normalize, projection_dim
        self.projection: nn.Module | None = None

    def forward(self, student_features: torch.Tensor, teacher_features: torch.Tensor) -> torch.Tensor:
        s, t = student_features, teacher_features.detach()
        if self.projection is None and s.shape[-1] != t.shape[-1]:
            self.projection = nn.Linear(s.shape[-1], self.projection_dim or t.shape[-1], bias=False).to(s.device, s.dtype)
        if self.projection is not None:
            s = self.projection(s)
        if self.normalize:
            s, t = F.normalize(s, dim=-1), F.normalize(t, dim=-1)
        if self.loss_type == "mse":
            return F.mse_loss(s, t)
        if self.loss_type == "l1":
            return F.l1_loss(s, t)
        return (1 - F.cosine_similarity(s, t, dim=-1)).mean()


class AttentionDistillationLoss(nn.Module):
    """Attention transfer: `mse` between the maps [B, H, Sq, Sk], or `kl` between their temperature-softened rows."""

    def __init__(self, loss_type: str = "mse", temperature: float = 1.0):
        super().__init__()
        if loss_type not in ("mse", "kl"):
            raise ValueError(f"unknown loss_type {loss_type!r}")
        self.loss_type, self.temperature = loss_type, temperature

    def forward(self, student_attention: torch.Tensor, teacher_attention: torch.Tensor) -> torch.Tensor:
        t = teacher_attention.detach()
        if self.loss_type == "mse":
            return F.mse_loss(student_attention, t)
        rows = student_attention.shape[-1]
        ls = F.log_softmax(student_attention.reshape(-1, rows) / self.temperature, dim=-1)
        pt = F.softmax(t.reshape(-1, rows) / self.temperature, dim=-1)
        return F.kl_div(ls, pt, reduction="batchmean")


class CharbonnierLoss(nn.Module):
    """sqrt((pred - target)^2 + eps^2): an L1 that is smooth at zero."""

    def __init__(self, epsilon: float = 1e-3, reduction: str = "mean"):
        super().__init__()
        self.epsilon, self.reduction = epsilon, reduction

    def forward(self, pred, target):
        return _reduce(torch.sqrt((pred - target).pow(2) + self.epsilon ** 2), self.reduction)


class PerceptualLoss(nn.Module):
    """MSE between the features a frozen network extracts from prediction and target.  The extractor may return one
    tensor or a dict of named feature maps; `layer_weights` picks and weights the named ones."""

    def __init__(self, feature_extractor: nn.Module, layer_weights: dict | None = None, normalize: bool = True):
        super().__init__()
        self.feature_extractor = feature_extractor.eval()
        for p in self.feature_extractor.parameters():
            p.requires_grad_(False)
        self.layer_weights = layer_weights or {"default": 1.0}
        self.normalize = normalize

    def forward(self, pred, target):
        with torch.no_grad():
            ft = self.feature_extractor(target)
        fp = self.feature_extractor(pred)
        if isinstance(fp, torch.Tensor):
            fp, ft = {"default": fp}, {"default": ft}
        total = pred.new_zeros(())
        for name, weight in self.layer_weights.items():
            if name not in fp:
                continue
            a, b = fp[name], ft[name].detach()
            if self.normalize:
                a, b = F.normalize(a, dim=1), F.normalize(b, dim=1)
            total = total + weight * F.mse_loss(a, b)
        return total


class ListMLELoss(nn.Module):
    """Listwise ranking: negative log-likelihood of the permutation that sorts the list by relevance under the
    Plackett-Luce model, -sum_i (s_i - logsumexp(s_i, ..., s_n)) over the scores in ideal order."""

    def __init__(self, eps: float = 1e-10, reduction: str = "mean"):
        super().__init__()
        self.eps, self.reduction = eps, reduction

    def forward(self, scores, relevance):
        order = relevance.argsort(dim=1, descending=True, stable=True)
        s = scores.gather(1, order)
        suffix_lse = torch.logcumsumexp(s.flip(1), dim=1).flip(1)       # logsumexp over positions i..n-1
        return _reduce(-(s - suffix_lse).sum(1), self.reduction)


class LambdaRankLoss(nn.Module):
    """Pairwise logistic (RankNet) loss with every pair weighted by the |change in NDCG| its swap would cause at the
    current ranking; averaged over the n(n-1)/2 pairs of a list."""

    def __init__(self, sigma: float = 1.0, reduction: str = "mean"):
        super().__init__()
        self.sigma, self.reduction = sigma, reduction

    @staticmethod
    def delta_ndcg(relevance: torch.Tensor, ranks: torch.Tensor) -> torch.Tensor:
        """[B, n, n]: |gain_i - gain_j| * |disc_i - disc_j| / IDCG with gain = 2^rel - 1, disc = 1 / log2(rank + 2)."""
        n = relevance.shape[1]
        gains = torch.pow(2.0, relevance.float()) - 1.0
        disc = 1.0 / torch.log2(ranks.float() + 2.0)
        ideal = 1.0 / torch.log2(torch.arange(n, device=relevance.device).float() + 2.0)
        idcg = (gains.sort(dim=1, descending=True).values * ideal).sum(1).clamp(min=1e-8)
        d = (gains.unsqueeze(2) - gains.unsqueeze(1)).abs() * (disc.unsqueeze(2) - disc.unsqueeze(1)).abs()
        return d / idcg.view(-1, 1, 1)

    def forward(self, scores, relevance):
        n = scores.shape[1]
        ranks = scores.argsort(dim=1, descending=True).argsort(dim=1)          # position of every item
        w = self.delta_ndcg(relevance, ranks)
        sign = torch.sign(relevance.unsqueeze(2).float() - relevance.unsqueeze(1).float())
        diff = scores.unsqueeze(2) - scores.unsqueeze(1)
        pair = w * F.softplus(-self.sigma * sign * diff)
        upper = torch.ones(n, n, device=scores.device).triu(1)
        return _reduce((pair * upper).sum((1, 2)) / upper.sum().clamp(min=1), self.reduction)


def _overlap(pred, target):
    p, t = pred.flatten(2), target.flatten(2).to(pred.dtype)
    tp = (p * t).sum(-1)
    return tp, (p * (1 - t)).sum(-1), ((1 - p) * t).sum(-1)


class FocalTverskyLoss(nn.Module):
    """(1 - Tversky index)^gamma per class on soft predictions [B, C, ...]; alpha weighs false positives, beta false
    negatives."""

    def __init__(self, alpha: float = 0.7, beta: float = 0.3, gamma: float = 0.75, smooth: float = 1.0,
                 reduction: str = "mean"):
        super().__init__()
        self.alpha, self.beta, self.gamma, self.smooth, self.reduction = alpha, beta, gamma, smooth, reduction

    def forward(self, pred, target):
        tp, fp, fn = _overlap(pred, target)
        tversky = (tp + self.smooth) / (tp + self.alpha * fp + self.beta * fn + self.smooth)
        return _reduce((1.0 - tversky).pow(self.gamma).mean(1), self.reduction)


class IoULoss(nn.Module):
    """1 - soft intersection-over-union per class on predictions [B, C, ...]."""

    def __init__(self, smooth: float = 1.0, reduction: str = "mean"):
        super().__init__()
        self.smooth, self.reduction = smooth, reduction

    def forward(self, pred, target):
        p, t = pred.flatten(2), target.flatten(2).to(pred.dtype)
        inter = (p * t).sum(-1)
        union = p.sum(-1) + t.sum(-1) - inter
        return _reduce((1.0 - (inter + self.smooth) / (union + self.smooth)).mean(1), self.reduction)


class BoundaryLoss(nn.Module):
    """Soft predictions [B, C, H, W] weighted by a precomputed signed distance map to the true boundary."""

    def __init__(self, reduction: str = "mean"):
        super().__init__()
        self.reduction = reduction

    def forward(self, pred, dist_map):
        return _reduce((pred * dist_map).sum((2, 3)).mean(1), self.reduction)


class GHMCLoss(nn.Module):
    """Gradient-harmonised classification loss: every example's cross-entropy is weighted by the inverse density of
    its gradient magnitude g = 1 - p(true class), estimated with a histogram of `bins` bins over [0, 1] (optionally an
    exponential moving average of the counts), so neither the mass of easy examples nor a few outliers dominate.
    Multi-class logits [B, C, ...] with class indices (or one-hot targets), or binary logits with 0 / 1 targets of the
    same shape; `mask` selects the valid examples."""

    def __init__(self, bins: int = 10, momentum: float = 0.0, reduction: str = "mean"):
        super().__init__()
        self.bins, self.momentum, self.reduction = bins, momentum, reduction
        self.register_buffer("edges", torch.linspace(0.0, 1.0, bins + 1))
        if momentum > 0:
            self.register_buffer("acc_sum", torch.zeros(bins))

    def forward(self, pred, target, mask=None):
        if pred.dim() > target.dim():
            p_true = F.softmax(pred, dim=1).gather(1, target.unsqueeze(1)).squeeze(1)
            base = F.cross_entropy(pred, target, reduction="none")
        else:
            sig = torch.sigmoid(pred)
            p_true = torch.where(target == 1, sig, 1 - sig)
            base = F.binary_cross_entropy_with_logits(pred, target.to(pred.dtype), reduction="none")
        g = (1 - p_true).detach()
        valid = torch.ones_like(g, dtype=torch.bool) if mask is None else mask.reshape(g.shape).bool()
        idx = torch.bucketize(g, self.edges[1:-1].to(g.device), right=True)          # bin of every example, 0..bins-1
        counts = torch.zeros(self.bins, device=g.device).index_add_(0, idx[valid].reshape(-1),
                                                                   torch.ones_like(g[valid]).reshape(-1).float())
        if self.momentum > 0:
            self.acc_sum = self.momentum * self.acc_sum.to(g.device) + (1 - self.momentum) * counts
            counts = self.acc_sum
        n = valid.sum().clamp(min=1).float()
        weights = (n / (counts.clamp(min=1) * self.bins))[idx] * valid.to(base.dtype)
        loss = base * weights
        if self.reduction == "mean":
            return loss.sum() / n if mask is not None else loss.mean()
        return _reduce(loss, self.reduction)


def create_label_smoothing_matrix(vocab_size: int, smoothing: float, device=None) -> torch.Tensor:
    """[V, V] soft targets of label smoothing: 1 - smoothing on the diagonal, smoothing / V everywhere else."""
    m = torch.full((vocab_size, vocab_size), smoothing / vocab_size, device=device)
    m.fill_diagonal_(1.0 - smoothing)
    return m
