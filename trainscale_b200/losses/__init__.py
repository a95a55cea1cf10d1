"""Loss library: language-model, preference, distillation, contrastive, MoE-auxiliary, regression / ranking /
segmentation losses, a registry and composition helpers.

Formulas follow data_pipeline/trainer/loss/__init__.py:130-521 and data_pipeline/trainer/loss/sota_losses.py:539-3268:
DPO `-log sigmoid(beta[(pi_c - pi_r) - (ref_c - ref_r)])` with hinge / IPO / robust variants and label smoothing
(:1190-1279), SimPO `-log sigmoid(beta(pi_c/|c| - pi_r/|r|) - gamma)` (:1478-1520), ORPO `nll + alpha * -log sigmoid(
log-odds ratio)` (:1394-1445), KTO with a detached batch-mean KL baseline (:1312-1363), CPO (:1542), distillation
`alpha T^2 KL + (1-alpha) CE` (:947-1022), MoE z-loss / load-balancing (:1993-2117).
On CUDA bf16 inputs the language-model losses run on the fused lm_head + cross-entropy kernels (ops/cross_entropy.py).
"""
from __future__ import annotations

import math
from typing import Callable, Mapping, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import cross_entropy as ce_ops
from ..utils.explicit_backward import ExplicitBackward as _ExplicitBackward


# ------------------------------------------------------------------------------------------------ helpers
def compute_log_probs(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                      average: bool = False, per_token: bool = False) -> torch.Tensor:
    """Per-sequence sum (or mean) of label-token log-probs; with `per_token` the [B, S] values themselves (0 at ignored
    positions).  logits [B,S,V] and labels [B,S] already aligned."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    mask = labels != ignore_index
    tok = lp.gather(-1, labels.clamp(min=0).unsqueeze(-1)).squeeze(-1) * mask
    if per_token:
        return tok
    s = tok.sum(-1)
    return s / mask.sum(-1).clamp(min=1) if average else s


def sequence_log_probs_from_hidden(hidden, weight, labels, ignore_index: int = -100, shift: bool = True):
    """(sum of log-probs [B], token counts [B]) straight from hidden states with the fused log-prob kernel."""
    if shift:
        tgt = torch.full_like(labels, ignore_index)
        tgt[..., :-1] = labels[..., 1:]
    else:
        tgt = labels
    lp = ce_ops.fused_linear_token_logprobs(hidden, weight, tgt, ignore_index)
    return lp.sum(-1), (tgt != ignore_index).sum(-1)


def get_sequence_lengths(labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    return (labels != ignore_index).sum(-1)


def _reduce(x: torch.Tensor, reduction: str) -> torch.Tensor:
    if reduction == "mean":
        return x.mean()
    if reduction == "sum":
        return x.sum()
    return x


# ------------------------------------------------------------------------------------------------ LM losses
class CrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index: int = -100, label_smoothing: float = 0.0, reduction: str = "mean",
                 z_loss_weight: float = 0.0):
        super().__init__()
        self.ignore_index, self.label_smoothing, self.reduction, self.z = ignore_index, label_smoothing, reduction, z_loss_weight

    def forward(self, logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        logits = logits.reshape(-1, logits.shape[-1]).float()
        labels = labels.reshape(-1)
        loss = F.cross_entropy(logits, labels, ignore_index=self.ignore_index, label_smoothing=self.label_smoothing,
                               reduction="sum" if self.reduction == "mean" else self.reduction)
        if self.reduction == "mean":
            loss = loss / (labels != self.ignore_index).sum().clamp(min=1)
        if self.z > 0:
            valid = labels != self.ignore_index
            loss = loss + self.z * (torch.logsumexp(logits[valid], -1) ** 2).mean()
        return loss


class FusedCrossEntropyLoss(_ExplicitBackward, CrossEntropyLoss):
    """Same contract; CUDA bf16 logits go through the row kernel (loss + lse in one pass)."""

    def forward(self, logits, labels):
        if logits.is_cuda and logits.dtype == torch.bfloat16 and self.z == 0 and self.reduction in ("mean", "sum"):
            z = logits.reshape(-1, logits.shape[-1])
            # forward and backward both run on the row kernel (FusedCrossEntropyFunction)
            rows = ce_ops.cross_entropy_rows(z, labels.reshape(-1), self.ignore_index, self.label_smoothing)
            s = rows.sum()
            return s / (labels != self.ignore_index).sum().clamp(min=1) if self.reduction == "mean" else s
        return super().forward(logits, labels)


FusedCrossEntropyFunction = ce_ops.FusedCrossEntropyFunction
Fast_CrossEntropyLoss = FusedCrossEntropyLoss      # name used by data_pipeline/trainer/kernels/triton_kernels.py:330


class ChunkedCrossEntropyLoss(nn.Module):
    """CE from hidden states without materialising [tokens, vocab]: `forward(hidden, lm_head_weight, labels)`."""

    def __init__(self, chunk_size: int = 4096, ignore_index: int = -100, label_smoothing: float = 0.0,
                 reduction: str = "mean", softcap: float = 0.0):
        super().__init__()
        self.chunk_size, self.ignore_index, self.label_smoothing = chunk_size, ignore_index, label_smoothing
        self.reduction, self.softcap = reduction, softcap

    def forward(self, hidden, weight, labels):
        loss, _ = ce_ops.fused_linear_cross_entropy(hidden, weight, labels.reshape(-1), self.ignore_index,
                                                    self.label_smoothing, 1.0, self.softcap,
                                                    min(self.chunk_size, 8192), self.reduction)
        return loss


class FocalLoss(nn.Module):
    def __init__(self, gamma: float = 2.0, alpha: float | None = 0.25, ignore_index: int = -100, reduction="mean"):
        super().__init__()
        self.gamma, self.alpha, self.ignore_index, self.reduction = gamma, alpha, ignore_index, reduction

    def forward(self, logits, labels):
        if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.shape[-1] % 8 == 0:
            # row kernel: online log-sum-exp forward, (softmax - onehot) * row scale backward, nothing V-wide in fp32
            from ..ops.cross_entropy import focal_loss_rows
            lab = labels.reshape(-1)
            loss = focal_loss_rows(logits.reshape(-1, logits.shape[-1]), lab, self.gamma, self.ignore_index)
            loss = loss[lab != self.ignore_index]
            if self.alpha is not None:
                loss = self.alpha * loss
            return _reduce(loss, self.reduction) if loss.numel() else logits.sum() * 0
        logits = logits.reshape(-1, logits.shape[-1]).float()
        labels = labels.reshape(-1)
        valid = labels != self.ignore_index
        logp = torch.log_softmax(logits[valid], -1).gather(1, labels[valid].unsqueeze(1)).squeeze(1)
        p = logp.exp()
        loss = -((1 - p) ** self.gamma) * logp
        if self.alpha is not None:
            loss = self.alpha * loss
        return _reduce(loss, self.reduction) if loss.numel() else logits.sum() * 0


class PolyLoss(nn.Module):
    """CE + epsilon * (1 - p_t)."""

    def __init__(self, epsilon: float = 1.0, ignore_index: int = -100):
        super().__init__()
        self.epsilon, self.ignore_index = epsilon, ignore_index

    def forward(self, logits, labels):
        if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.shape[-1] % 8 == 0:
            # row kernel: online log-sum-exp forward, (softmax - onehot) * row scale backward, nothing V-wide in fp32
            from ..ops.cross_entropy import focal_loss_rows
            lab = labels.reshape(-1)
            loss = focal_loss_rows(logits.reshape(-1, logits.shape[-1]), lab, self.gamma, self.ignore_index)
            loss = loss[lab != self.ignore_index]
            if self.alpha is not None:
                loss = self.alpha * loss
            return _reduce(loss, self.reduction) if loss.numel() else logits.sum() * 0
        logits = logits.reshape(-1, logits.shape[-1]).float()
        labels = labels.reshape(-1)
        valid = labels != self.ignore_index
        logp = torch.log_softmax(logits[valid], -1).gather(1, labels[valid].unsqueeze(1)).squeeze(1)
        return (-logp + self.epsilon * (1 - logp.exp())).mean()


class KLDivergenceLoss(nn.Module):
    def __init__(self, temperature: float = 1.0, reduction: str = "batchmean", log_target: bool = False):
        super().__init__()
        self.t, self.reduction, self.log_target = temperature, reduction, log_target

    def forward(self, student_logits, teacher_logits):
        s = torch.log_softmax(student_logits.float() / self.t, -1)
        t = torch.log_softmax(teacher_logits.float() / self.t, -1) if self.log_target else torch.softmax(teacher_logits.float() / self.t, -1)
        return F.kl_div(s.reshape(-1, s.shape[-1]), t.reshape(-1, t.shape[-1]), reduction=self.reduction,
                        log_target=self.log_target) * self.t ** 2


class DistillationLoss(nn.Module):
    def __init__(self, temperature: float = 2.0, alpha: float = 0.5, ignore_index: int = -100):
        super().__init__()
        self.t, self.alpha, self.ignore_index = temperature, alpha, ignore_index

    def forward(self, student_logits, teacher_logits, labels=None):
        V = student_logits.shape[-1]
        s, t = student_logits.reshape(-1, V).float(), teacher_logits.reshape(-1, V).float()
        if labels is not None:
            valid = labels.reshape(-1) != self.ignore_index
            s_v, t_v = s[valid], t[valid]
        else:
            s_v, t_v = s, t
        kd = F.kl_div(torch.log_softmax(s_v / self.t, -1), torch.softmax(t_v / self.t, -1), reduction="batchmean") * self.t ** 2
        if labels is None:
            return kd
        ce = F.cross_entropy(s, labels.reshape(-1), ignore_index=self.ignore_index)
        return self.alpha * kd + (1 - self.alpha) * ce


# ------------------------------------------------------------------------------------------------ preference losses
class DPOLoss(nn.Module):
    """Inputs are per-sequence summed log-probs. Returns (loss, chosen_rewards, rejected_rewards)."""

    def __init__(self, beta: float = 0.1, loss_type: str = "sigmoid", label_smoothing: float = 0.0,
                 reference_free: bool = False):
        super().__init__()
        self.beta, self.loss_type, self.label_smoothing, self.reference_free = beta, loss_type, label_smoothing, reference_free

    def forward(self, policy_chosen, policy_rejected, ref_chosen=None, ref_rejected=None):
        pi = policy_chosen - policy_rejected
        ref = 0.0 if (self.reference_free or ref_chosen is None) else (ref_chosen - ref_rejected)
        x = pi - ref
        b, eps = self.beta, self.label_smoothing
        if self.loss_type == "sigmoid":
            loss = -F.logsigmoid(b * x) * (1 - eps) - F.logsigmoid(-b * x) * eps
        elif self.loss_type == "robust":
            loss = (-F.logsigmoid(b * x) * (1 - eps) + F.logsigmoid(-b * x) * eps) / (1 - 2 * eps)
        elif self.loss_type == "hinge":
            loss = torch.relu(1 - b * x)
        elif self.loss_type == "ipo":
            loss = (x - 1 / (2 * b)) ** 2
        elif self.loss_type == "kto_pair":
            ck = (policy_chosen - (ref_chosen if ref_chosen is not None else 0)).mean().clamp(min=0).detach()
            rk = (policy_rejected - (ref_rejected if ref_rejected is not None else 0)).mean().clamp(min=0).detach()
            cl = policy_chosen - (ref_chosen if ref_chosen is not None else 0)
            rl = policy_rejected - (ref_rejected if ref_rejected is not None else 0)
            loss = torch.cat((1 - torch.sigmoid(b * (cl - rk)), 1 - torch.sigmoid(b * (ck - rl))))
        else:
            raise ValueError(f"unknown DPO loss type {self.loss_type!r}")
        rc = b * (policy_chosen - (ref_chosen if ref_chosen is not None and not self.reference_free else 0)).detach()
        rr = b * (policy_rejected - (ref_rejected if ref_rejected is not None and not self.reference_free else 0)).detach()
        return loss.mean(), rc, rr

    @staticmethod
    def accuracy(chosen_rewards, rejected_rewards) -> torch.Tensor:
        return (chosen_rewards > rejected_rewards).float().mean()


class SimPOLoss(nn.Module):
    """Length-normalised, reference-free."""

    def __init__(self, beta: float = 2.0, gamma: float = 0.5, label_smoothing: float = 0.0):
        super().__init__()
        self.beta, self.gamma, self.eps = beta, gamma, label_smoothing

    def forward(self, policy_chosen, policy_rejected, chosen_lengths, rejected_lengths):
        c = policy_chosen / chosen_lengths.clamp(min=1)
        r = policy_rejected / rejected_lengths.clamp(min=1)
        x = self.beta * (c - r) - self.gamma
        loss = -F.logsigmoid(x) * (1 - self.eps) - F.logsigmoid(-x) * self.eps
        return loss.mean(), (self.beta * c).detach(), (self.beta * r).detach()


class ORPOLoss(nn.Module):
    """Inputs are AVERAGE per-token log-probs; nll_chosen is the SFT loss on the chosen answers."""

    def __init__(self, alpha: float = 0.1):
        super().__init__()
        self.alpha = alpha

    @staticmethod
    def log_odds(logp):
        return logp - torch.log1p(-torch.exp(logp).clamp(max=1 - 1e-7))

    def forward(self, avg_logp_chosen, avg_logp_rejected, nll_chosen):
        ratio = self.log_odds(avg_logp_chosen) - self.log_odds(avg_logp_rejected)
        pref = -F.logsigmoid(ratio).mean()
        return nll_chosen + self.alpha * pref, ratio.detach()


class KTOLoss(nn.Module):
    def __init__(self, beta: float = 0.1, desirable_weight: float = 1.0, undesirable_weight: float = 1.0):
        super().__init__()
        self.beta, self.wd, self.wu = beta, desirable_weight, undesirable_weight

    def forward(self, policy_logps, ref_logps, is_desirable: torch.Tensor):
        r = policy_logps - ref_logps
        kl = r.mean().clamp(min=0).detach()
        d = is_desirable.bool()
        loss_d = 1 - torch.sigmoid(self.beta * (r - kl))
        loss_u = 1 - torch.sigmoid(self.beta * (kl - r))
        loss = torch.where(d, self.wd * loss_d, self.wu * loss_u)
        return loss.mean(), (self.beta * r).detach()


class CPOLoss(nn.Module):
    """Contrastive preference optimisation: reference-free DPO term + NLL on the chosen answer."""

    def __init__(self, beta: float = 0.1, alpha: float = 1.0, label_smoothing: float = 0.0):
        super().__init__()
        self.beta, self.alpha, self.eps = beta, alpha, label_smoothing

    def forward(self, policy_chosen, policy_rejected, nll_chosen):
        x = self.beta * (policy_chosen - policy_rejected)
        pref = (-F.logsigmoid(x) * (1 - self.eps) - F.logsigmoid(-x) * self.eps).mean()
        return pref + self.alpha * nll_chosen


# ------------------------------------------------------------------------------------------------ contrastive
def _gather_embeddings(x: torch.Tensor) -> torch.Tensor:
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
        return x
    parts = [torch.zeros_like(x) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, x.contiguous())
    parts[dist.get_rank()] = x   # keep the autograd path of the local shard
    return torch.cat(parts)


class InfoNCELoss(nn.Module):
    def __init__(self, temperature: float = 0.07, gather: bool = False):
        super().__init__()
        self.t, self.gather = temperature, gather

    def forward(self, query, key):
        q, k = F.normalize(query.float(), dim=-1), F.normalize(key.float(), dim=-1)
        if self.gather:
            k = _gather_embeddings(k)
        logits = q @ k.t() / self.t
        off = 0
        if self.gather and k.shape[0] != q.shape[0]:
            import torch.distributed as dist
            off = dist.get_rank() * q.shape[0]
        return F.cross_entropy(logits, torch.arange(q.shape[0], device=q.device) + off)


class CLIPLoss(nn.Module):
    def __init__(self, init_temperature: float = 0.07, learnable: bool = True):
        super().__init__()
        t = torch.tensor(math.log(1 / init_temperature))
        self.logit_scale = nn.Parameter(t) if learnable else t

    @property
    def temperature(self) -> torch.Tensor:
        """Current soft-max temperature, 1 / exp(logit_scale) (the scale itself is capped at 100)."""
        return 1.0 / self.logit_scale.exp().clamp(max=100)

    def forward(self, image_emb, text_emb):
        a, b = F.normalize(image_emb.float(), dim=-1), F.normalize(text_emb.float(), dim=-1)
        logits = self.logit_scale.exp().clamp(max=100) * a @ b.t()
        tgt = torch.arange(a.shape[0], device=a.device)
        return 0.5 * (F.cross_entropy(logits, tgt) + F.cross_entropy(logits.t(), tgt))


class TripletLoss(nn.Module):
    def __init__(self, margin: float = 1.0, distance: str = "euclidean"):
        super().__init__()
        self.margin, self.distance = margin, distance

    def forward(self, anchor, positive, negative):
        if self.distance == "cosine":
            dp, dn = 1 - F.cosine_similarity(anchor, positive), 1 - F.cosine_similarity(anchor, negative)
        else:
            dp, dn = F.pairwise_distance(anchor, positive), F.pairwise_distance(anchor, negative)
        return torch.relu(dp - dn + self.margin).mean()


class NTXentLoss(nn.Module):
    def __init__(self, temperature: float = 0.5):
        super().__init__()
        self.t = temperature

    def forward(self, z1, z2):
        n = z1.shape[0]
        z = F.normalize(torch.cat((z1, z2)).float(), dim=-1)
        sim = z @ z.t() / self.t
        sim.fill_diagonal_(float("-inf"))
        tgt = torch.cat((torch.arange(n, 2 * n), torch.arange(0, n))).to(z.device)
        return F.cross_entropy(sim, tgt)


class SupConLoss(nn.Module):
    def __init__(self, temperature: float = 0.07):
        super().__init__()
        self.t = temperature

    def forward(self, features, labels):
        z = F.normalize(features.float(), dim=-1)
        sim = z @ z.t() / self.t
        eye = torch.eye(z.shape[0], dtype=torch.bool, device=z.device)
        sim = sim.masked_fill(eye, float("-inf"))
        pos = (labels.unsqueeze(0) == labels.unsqueeze(1)) & ~eye
        logp = sim - torch.logsumexp(sim, dim=1, keepdim=True)
        n_pos = pos.sum(1)
        loss = -(logp.masked_fill(~pos, 0).sum(1) / n_pos.clamp(min=1))
        return loss[n_pos > 0].mean() if (n_pos > 0).any() else sim.sum() * 0


# ------------------------------------------------------------------------------------------------ MoE auxiliary
class ZLoss(nn.Module):
    def __init__(self, weight: float = 1e-3):
        super().__init__()
        self.weight = weight

    def forward(self, router_logits):
        return self.weight * (torch.logsumexp(router_logits.float(), dim=-1) ** 2).mean()


class LoadBalancingLoss(nn.Module):
    """E * sum_i f_i P_i (f = fraction of tokens routed to expert i, P = mean router probability)."""

    def __init__(self, num_experts: int, top_k: int = 1, weight: float = 1e-2):
        super().__init__()
        self.E, self.k, self.weight = num_experts, top_k, weight

    def forward(self, router_logits, expert_indices=None):
        probs = torch.softmax(router_logits.float().reshape(-1, self.E), -1)
        if expert_indices is None:
            expert_indices = probs.topk(self.k, dim=-1).indices
        f = F.one_hot(expert_indices.reshape(-1), self.E).float().mean(0) * 1.0
        return self.weight * self.E * (f * probs.mean(0)).sum()


class ExpertEntropyLoss(nn.Module):
    def __init__(self, weight: float = 1e-3):
        super().__init__()
        self.weight = weight

    def forward(self, router_logits):
        p = torch.softmax(router_logits.float(), -1).reshape(-1, router_logits.shape[-1]).mean(0)
        return -self.weight * -(p * (p + 1e-9).log()).sum()   # maximise usage entropy


# ------------------------------------------------------------------------------------------------ regression / ranking / segmentation
class MSELoss(nn.MSELoss): ...
class MAELoss(nn.L1Loss): ...
class HuberLoss(nn.HuberLoss): ...
class SmoothL1Loss(nn.SmoothL1Loss): ...


class LogCoshLoss(nn.Module):
    def forward(self, pred, target):
        d = pred - target
        return (d + F.softplus(-2 * d) - math.log(2.0)).mean()


class QuantileLoss(nn.Module):
    def __init__(self, quantile: float = 0.5):
        super().__init__()
        self.q = quantile

    def forward(self, pred, target):
        d = target - pred
        return torch.max(self.q * d, (self.q - 1) * d).mean()


class MarginRankingLoss(nn.MarginRankingLoss): ...


class ListNetLoss(nn.Module):
    def forward(self, scores, relevance):
        return -(torch.softmax(relevance.float(), -1) * torch.log_softmax(scores.float(), -1)).sum(-1).mean()


class PairwiseRewardLoss(nn.Module):
    """Bradley-Terry reward-model loss: -log sigmoid(r_chosen - r_rejected - margin)."""

    def __init__(self, margin: float = 0.0):
        super().__init__()
        self.margin = margin

    def forward(self, chosen_reward, rejected_reward):
        return -F.logsigmoid(chosen_reward - rejected_reward - self.margin).mean()


class DiceLoss(nn.Module):
    def __init__(self, smooth: float = 1.0):
        super().__init__()
        self.smooth = smooth

    def forward(self, logits, target):
        p = torch.sigmoid(logits.float()).flatten(1)
        t = target.float().flatten(1)
        inter = (p * t).sum(1)
        return (1 - (2 * inter + self.smooth) / (p.sum(1) + t.sum(1) + self.smooth)).mean()


class TverskyLoss(nn.Module):
    def __init__(self, alpha: float = 0.5, beta: float = 0.5, smooth: float = 1.0):
        super().__init__()
        self.a, self.b, self.smooth = alpha, beta, smooth

    def forward(self, logits, target):
        p, t = torch.sigmoid(logits.float()).flatten(1), target.float().flatten(1)
        tp, fp, fn = (p * t).sum(1), (p * (1 - t)).sum(1), ((1 - p) * t).sum(1)
        return (1 - (tp + self.smooth) / (tp + self.a * fp + self.b * fn + self.smooth)).mean()


class BCEWithLogitsLoss(nn.BCEWithLogitsLoss): ...


from .extra import (AttentionDistillationLoss, BoundaryLoss, CharbonnierLoss, FeatureDistillationLoss,  # noqa: E402
                    FocalTverskyLoss, GHMCLoss, IoULoss, LambdaRankLoss, ListMLELoss, LossOutput, PerceptualLoss,
                    create_label_smoothing_matrix)


# ------------------------------------------------------------------------------------------------ registry / composition
class LossRegistry:
    _losses: dict[str, Callable[..., nn.Module]] = {}

    @classmethod
    def register(cls, name: str, factory: Callable[..., nn.Module] | None = None):
        if factory is not None:
            cls._losses[name] = factory
            return factory

        def deco(f):
            cls._losses[name] = f
            return f
        return deco

    @classmethod
    def create(cls, name: str, **kw) -> nn.Module:
        if name not in cls._losses:
            raise KeyError(f"unknown loss {name!r}; available: {sorted(cls._losses)}")
        return cls._losses[name](**kw)

    @classmethod
    def available(cls) -> list[str]:
        return sorted(cls._losses)

    # the reference's names for the same two calls (data_pipeline/trainer/loss/sota_losses.py:2909-3000)
    get = create
    list_available = available


for _n, _c in {"cross_entropy": CrossEntropyLoss, "fused_cross_entropy": FusedCrossEntropyLoss,
               "chunked_ce": ChunkedCrossEntropyLoss, "focal": FocalLoss, "poly": PolyLoss, "kl_div": KLDivergenceLoss,
               "distillation": DistillationLoss, "dpo": DPOLoss, "simpo": SimPOLoss, "orpo": ORPOLoss, "kto": KTOLoss,
               "cpo": CPOLoss, "infonce": InfoNCELoss, "contrastive": InfoNCELoss, "clip": CLIPLoss,
               "triplet": TripletLoss, "ntxent": NTXentLoss, "supcon": SupConLoss, "z_loss": ZLoss,
               "load_balancing": LoadBalancingLoss, "expert_entropy": ExpertEntropyLoss, "mse": MSELoss, "mae": MAELoss,
               "huber": HuberLoss, "smooth_l1": SmoothL1Loss, "log_cosh": LogCoshLoss, "quantile": QuantileLoss,
               "margin_ranking": MarginRankingLoss, "listnet": ListNetLoss, "pairwise_reward": PairwiseRewardLoss,
               "dice": DiceLoss, "tversky": TverskyLoss, "bce": BCEWithLogitsLoss,
               "feature_distillation": FeatureDistillationLoss, "attention_distillation": AttentionDistillationLoss,
               "charbonnier": CharbonnierLoss, "list_mle": ListMLELoss, "lambda_rank": LambdaRankLoss,
               "focal_tversky": FocalTverskyLoss, "ghmc": GHMCLoss, "iou": IoULoss, "boundary": BoundaryLoss}.items():
    LossRegistry.register(_n, _c)


class CompositeLoss(nn.Module):
    """Weighted sum of named losses; each entry is (loss, weight, argument names taken from the kwargs)."""

    def __init__(self, parts: Mapping[str, tuple[nn.Module, float, Sequence[str]]]):
        super().__init__()
        self.names = list(parts)
        self.mods = nn.ModuleList(p[0] for p in parts.values())
        self.weights = [p[1] for p in parts.values()]
        self.args = [list(p[2]) for p in parts.values()]

    def forward(self, **kw):
        total, detail = 0.0, {}
        for n, m, w, a in zip(self.names, self.mods, self.weights, self.args):
            v = m(*[kw[k] for k in a])
            v = v[0] if isinstance(v, tuple) else v
            detail[n] = v.detach()
            total = total + w * v
        return total, detail


class MultiTaskLoss(nn.Module):
    """Homoscedastic-uncertainty weighting: sum_i exp(-s_i) L_i + s_i."""

    def __init__(self, num_tasks: int):
        super().__init__()
        self.log_vars = nn.Parameter(torch.zeros(num_tasks))

    def forward(self, losses: Sequence[torch.Tensor]):
        return sum(torch.exp(-self.log_vars[i]) * l + self.log_vars[i] for i, l in enumerate(losses))


def create_loss(name: str = "cross_entropy", **kw) -> nn.Module:
    return LossRegistry.create(getattr(name, "value", name), **kw)


def create_loss_from_config(lc) -> nn.Module:
    """From a SOTAConfig `loss` section."""
    t = getattr(lc.type, "value", lc.type)
    if t in ("cross_entropy",):
        return FusedCrossEntropyLoss(lc.ignore_index, lc.label_smoothing, lc.reduction)
    if t == "chunked_ce":
        return ChunkedCrossEntropyLoss(lc.chunk_size, lc.ignore_index, lc.label_smoothing, lc.reduction)
    if t == "focal":
        return FocalLoss(lc.focal_gamma, lc.focal_alpha, lc.ignore_index, lc.reduction)
    if t == "dpo":
        return DPOLoss(lc.dpo_beta, getattr(lc, "dpo_variant", "sigmoid"), lc.label_smoothing,
                       getattr(lc, "reference_free", False))
    if t == "simpo":
        return SimPOLoss(lc.dpo_beta, getattr(lc, "simpo_gamma", 0.5), lc.label_smoothing)
    if t == "orpo":
        return ORPOLoss(lc.alpha)
    if t == "kto":
        return KTOLoss(lc.dpo_beta)
    if t == "cpo":
        return CPOLoss(lc.dpo_beta, lc.alpha, lc.label_smoothing)
    if t == "distillation":
        return DistillationLoss(lc.temperature, lc.alpha, lc.ignore_index)
    if t == "contrastive":
        return InfoNCELoss(lc.temperature if lc.temperature < 1 else 0.07)
    return create_loss(t)
