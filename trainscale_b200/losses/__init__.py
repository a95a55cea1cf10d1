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
from ..utils.refargs import ANY, reference_kwargs


# ------------------------------------------------------------------------------------------------ helpers
def _ref_output(_total: torch.Tensor, **metrics):
    """`LossOutput(loss, metrics)`: what the forward of a preference / composite loss returns when it is called with
    the reference's keyword names (data_pipeline/trainer/loss/sota_losses.py); this framework's own calling forms keep
    returning tensors / tuples."""
    from .extra import LossOutput
    return LossOutput(_total, {k: float(v.detach()) if torch.is_tensor(v) else float(v) for k, v in metrics.items()})


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
    @reference_kwargs({"use_triton": ANY})
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


class ChunkedCrossEntropyLoss(nn.Module):
    """CE from hidden states without materialising [tokens, vocab]: `forward(hidden, lm_head_weight, labels)`."""

    def __init__(self, chunk_size: int = 4096, ignore_index: int = -100, label_smoothing: float = 0.0,
                 reduction: str = "mean", softcap: float = 0.0):
        super().__init__()
        self.chunk_size, self.ignore_index, self.label_smoothing = chunk_size, ignore_index, label_smoothing
        self.reduction, self.softcap = reduction, softcap

    def forward(self, hidden=None, weight=None, labels=None, *, logits=None):
        """`forward(hidden, lm_head_weight, labels)` never builds the logits.  The reference's `forward(logits, labels)`
        (data_pipeline/trainer/loss/sota_losses.py ChunkedCrossEntropyLoss) takes logits that already exist and walks
        them in row chunks of `chunk_size`, so that only one chunk is upcast at a time."""
        if logits is not None or labels is None:
            logits, labels = (logits if logits is not None else hidden), (labels if labels is not None else weight)
            z, y = logits.reshape(-1, logits.shape[-1]), labels.reshape(-1)
            rows = torch.cat([F.cross_entropy(z[i:i + self.chunk_size].float(), y[i:i + self.chunk_size],
                                              ignore_index=self.ignore_index, label_smoothing=self.label_smoothing,
                                              reduction="none") for i in range(0, z.shape[0], self.chunk_size)])
            if self.reduction == "none":
                return rows.view(labels.shape)
            return rows.sum() / (y != self.ignore_index).sum().clamp(min=1) if self.reduction == "mean" else rows.sum()
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

    def __init__(self, epsilon: float = 1.0, ignore_index: int = -100, reduction: str = "mean"):
        super().__init__()
        self.epsilon, self.ignore_index, self.reduction = epsilon, ignore_index, reduction

    def forward(self, logits, labels):
        logits = logits.reshape(-1, logits.shape[-1]).float()
        labels = labels.reshape(-1)
        valid = labels != self.ignore_index
        logp = torch.log_softmax(logits[valid], -1).gather(1, labels[valid].unsqueeze(1)).squeeze(1)
        loss = -logp + self.epsilon * (1 - logp.exp())
        return _reduce(loss, self.reduction) if loss.numel() else logits.sum() * 0


class KLDivergenceLoss(nn.Module):
    """KL(teacher || student) on temperature-softened distributions, times T^2.  `mode="reverse"` swaps the two
    (mode-seeking instead of mass-covering); `forward(input=, target=)` are the reference's names for the logits."""

    def __init__(self, temperature: float = 1.0, reduction: str = "batchmean", log_target: bool = False,
                 mode: str = "forward"):
        super().__init__()
        if mode not in ("forward", "reverse"):
            raise ValueError("mode must be 'forward' or 'reverse'")
        self.t, self.reduction, self.log_target, self.mode = temperature, reduction, log_target, mode

    @reference_kwargs(input="student_logits", target="teacher_logits")
    def forward(self, student_logits, teacher_logits):
        if self.mode == "reverse":
            student_logits, teacher_logits = teacher_logits, student_logits
        s = torch.log_softmax(student_logits.float() / self.t, -1)
        t = torch.log_softmax(teacher_logits.float() / self.t, -1) if self.log_target else torch.softmax(teacher_logits.float() / self.t, -1)
        return F.kl_div(s.reshape(-1, s.shape[-1]), t.reshape(-1, t.shape[-1]), reduction=self.reduction,
                        log_target=self.log_target) * self.t ** 2


class DistillationLoss(nn.Module):
    """alpha * T^2 KL(teacher || student) + (1 - alpha) CE.  `distill_type`: "soft" (that), "hard" (cross-entropy
    against the teacher's arg-max instead of the KL term)."""

    def __init__(self, temperature: float = 2.0, alpha: float = 0.5, ignore_index: int = -100, reduction: str = "mean",
                 distill_type: str = "soft"):
        super().__init__()
        if reduction not in ("mean", "batchmean"):
            raise ValueError("DistillationLoss reduces to a scalar: reduction must be 'mean'")
        self.t, self.alpha, self.ignore_index, self.distill_type = temperature, alpha, ignore_index, distill_type

    def forward(self, student_logits, teacher_logits, labels=None):
        V = student_logits.shape[-1]
        s, t = student_logits.reshape(-1, V).float(), teacher_logits.reshape(-1, V).float()
        if labels is not None:
            valid = labels.reshape(-1) != self.ignore_index
            s_v, t_v = s[valid], t[valid]
        else:
            s_v, t_v = s, t
        if self.distill_type == "hard":
            kd = F.cross_entropy(s_v, t_v.argmax(-1))
        else:
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

    @reference_kwargs(policy_chosen_logps="policy_chosen", policy_rejected_logps="policy_rejected",
                      reference_chosen_logps="ref_chosen", reference_rejected_logps="ref_rejected")
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

    @reference_kwargs(policy_chosen_logps="policy_chosen", policy_rejected_logps="policy_rejected",
                      chosen_length="chosen_lengths", rejected_length="rejected_lengths")
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

    @reference_kwargs(policy_chosen_logps="avg_logp_chosen", policy_rejected_logps="avg_logp_rejected",
                      chosen_nll_loss="nll_chosen")
    def forward(self, avg_logp_chosen, avg_logp_rejected, nll_chosen):
        ratio = self.log_odds(avg_logp_chosen) - self.log_odds(avg_logp_rejected)
        pref = -F.logsigmoid(ratio).mean()
        return nll_chosen + self.alpha * pref, ratio.detach()


class KTOLoss(nn.Module):
    def __init__(self, beta: float = 0.1, desirable_weight: float = 1.0, undesirable_weight: float = 1.0):
        super().__init__()
        self.beta, self.wd, self.wu = beta, desirable_weight, undesirable_weight

    @reference_kwargs(reference_logps="ref_logps")
    def forward(self, policy_logps, ref_logps, is_desirable: torch.Tensor, kl_baseline: torch.Tensor | None = None):
        """`kl_baseline`: the reference point z0 (a scalar or per-example tensor); by default the batch's mean log
        ratio, clamped at 0."""
        r = policy_logps - ref_logps
        kl = r.mean().clamp(min=0).detach() if kl_baseline is None else torch.as_tensor(kl_baseline).detach()
        d = is_desirable.bool()
        loss_d = 1 - torch.sigmoid(self.beta * (r - kl))
        loss_u = 1 - torch.sigmoid(self.beta * (kl - r))
        loss = torch.where(d, self.wd * loss_d, self.wu * loss_u)
        return loss.mean(), (self.beta * r).detach()


class CPOLoss(nn.Module):
    """Contrastive preference optimisation: reference-free DPO term + NLL on the chosen answer."""

    def __init__(self, beta: float = 0.1, alpha: float = 1.0, label_smoothing: float = 0.0, bc_coef: float | None = None):
        super().__init__()
        self.beta, self.alpha, self.eps = beta, (alpha if bc_coef is None else bc_coef), label_smoothing

    @property
    def bc_coef(self) -> float:
        """Weight of the behaviour-cloning (NLL on the chosen answer) term: the reference's name for `alpha`."""
        return self.alpha

    def forward(self, policy_chosen=None, policy_rejected=None, nll_chosen=None, *, policy_chosen_logps=None,
                policy_rejected_logps=None, reference_chosen_logps=None, reference_rejected_logps=None,
                chosen_nll_loss=None):
        """(policy_chosen, policy_rejected, nll_chosen) -> scalar.  The reference's keyword form subtracts the
        reference model's log ratio, takes several rejected answers per prompt ([B, R]) and returns `LossOutput`
        (data_pipeline/trainer/loss/sota_losses.py, CPOLoss.forward)."""
        if policy_chosen_logps is not None:
            rej = policy_rejected_logps if policy_rejected_logps.dim() > 1 else policy_rejected_logps.unsqueeze(1)
            pi = policy_chosen_logps.unsqueeze(1) - rej
            if reference_chosen_logps is not None:
                rr = reference_rejected_logps if reference_rejected_logps.dim() > 1 else reference_rejected_logps.unsqueeze(1)
                pi = pi - (reference_chosen_logps.unsqueeze(1) - rr)
            losses = -F.logsigmoid(self.beta * pi).mean(1)
            if self.alpha > 0 and chosen_nll_loss is not None:
                losses = losses + self.alpha * chosen_nll_loss
            return _ref_output(losses.mean(), loss=losses.mean(), accuracy=(pi > 0).float().mean())
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
    """query -> key contrastive loss with in-batch negatives.  The reference's form `forward(embeddings_a=,
    embeddings_b=, labels=)` is symmetric (mean of a->b and b->a) and takes custom positive indices."""

    @reference_kwargs(gather_distributed="gather")
    def __init__(self, temperature: float = 0.07, gather: bool = False, reduction: str = "mean"):
        super().__init__()
        self.t, self.gather, self.reduction = temperature, gather, reduction

    def forward(self, query=None, key=None, *, embeddings_a=None, embeddings_b=None, labels=None):
        if embeddings_a is not None:
            a, b = F.normalize(embeddings_a.float(), dim=-1), F.normalize(embeddings_b.float(), dim=-1)
            if self.gather:
                a, b = _gather_embeddings(a), _gather_embeddings(b)
            logits = a @ b.t() / self.t
            tgt = labels if labels is not None else torch.arange(a.shape[0], device=a.device)
            return 0.5 * (F.cross_entropy(logits, tgt, reduction=self.reduction)
                          + F.cross_entropy(logits.t(), tgt, reduction=self.reduction))
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
    @reference_kwargs(learnable_temperature="learnable")
    def __init__(self, init_temperature: float = 0.07, learnable: bool = True, max_temperature: float | None = None):
        """`max_temperature`: upper bound of the temperature (a lower bound of the logit scale); None = unbounded."""
        super().__init__()
        t = torch.tensor(math.log(1 / init_temperature))
        self.logit_scale = nn.Parameter(t) if learnable else t
        self.min_scale = None if max_temperature is None else 1.0 / max_temperature

    @property
    def temperature(self) -> torch.Tensor:
        """Current soft-max temperature, 1 / exp(logit_scale) (the scale itself is capped at 100)."""
        return 1.0 / self.logit_scale.exp().clamp(max=100)

    @reference_kwargs(image_embeddings="image_emb", text_embeddings="text_emb")
    def forward(self, image_emb, text_emb):
        a, b = F.normalize(image_emb.float(), dim=-1), F.normalize(text_emb.float(), dim=-1)
        logits = self.logit_scale.exp().clamp(min=getattr(self, "min_scale", None), max=100) * a @ b.t()
        tgt = torch.arange(a.shape[0], device=a.device)
        return 0.5 * (F.cross_entropy(logits, tgt) + F.cross_entropy(logits.t(), tgt))


class TripletLoss(nn.Module):
    """max(0, d(a, p) - d(a, n) + margin).  `hard_mining`: each anchor is paired with the hardest negative of the
    batch (the closest of all `negative` rows) instead of its own row."""

    def __init__(self, margin: float = 1.0, distance: str = "euclidean", hard_mining: bool = False,
                 reduction: str = "mean"):
        super().__init__()
        self.margin, self.distance, self.hard_mining, self.reduction = margin, distance, hard_mining, reduction

    def _dist(self, a, b):
        if self.distance == "cosine":
            return 1 - F.normalize(a, dim=-1) @ F.normalize(b, dim=-1).t()
        return torch.cdist(a, b)

    def forward(self, anchor, positive, negative):
        if self.hard_mining:
            dp = self._dist(anchor.float(), positive.float()).diagonal()
            dn = self._dist(anchor.float(), negative.float()).min(1).values
        elif self.distance == "cosine":
            dp, dn = 1 - F.cosine_similarity(anchor, positive), 1 - F.cosine_similarity(anchor, negative)
        else:
            dp, dn = F.pairwise_distance(anchor, positive), F.pairwise_distance(anchor, negative)
        return _reduce(torch.relu(dp - dn + self.margin), self.reduction)


class NTXentLoss(nn.Module):
    """SimCLR loss over two views.  `forward(z1, z2)`, or the reference's `forward(embeddings)` with the two views
    stacked along the batch, [2N, D]."""

    def __init__(self, temperature: float = 0.5, reduction: str = "mean"):
        super().__init__()
        self.t, self.reduction = temperature, reduction

    def forward(self, z1=None, z2=None, *, embeddings=None):
        if embeddings is not None or z2 is None:
            both = embeddings if embeddings is not None else z1
            n = both.shape[0] // 2
            z1, z2 = both[:n], both[n:]
        n = z1.shape[0]
        z = F.normalize(torch.cat((z1, z2)).float(), dim=-1)
        sim = z @ z.t() / self.t
        sim.fill_diagonal_(float("-inf"))
        tgt = torch.cat((torch.arange(n, 2 * n), torch.arange(0, n))).to(z.device)
        return F.cross_entropy(sim, tgt, reduction=self.reduction)


class SupConLoss(nn.Module):
    """Supervised contrastive loss.  `features`: [B, D] or [B, views, D] (labels are repeated per view); `mask`: an
    explicit [B, B] positive mask instead of label equality; the loss is scaled by temperature / base_temperature."""

    def __init__(self, temperature: float = 0.07, base_temperature: float | None = None, reduction: str = "mean"):
        super().__init__()
        self.t, self.base_t, self.reduction = temperature, base_temperature or temperature, reduction

    @reference_kwargs(embeddings="features")
    def forward(self, features, labels=None, mask=None):
        if features.dim() == 3:
            B, V, _ = features.shape
            features = features.transpose(0, 1).reshape(B * V, -1)           # view-major, like labels.repeat(V)
            labels = labels.repeat(V) if labels is not None else None
            mask = mask.repeat(V, V) if mask is not None else None
        z = F.normalize(features.float(), dim=-1)
        sim = z @ z.t() / self.t
        eye = torch.eye(z.shape[0], dtype=torch.bool, device=z.device)
        sim = sim.masked_fill(eye, float("-inf"))
        pos = (mask.bool() if mask is not None else labels.unsqueeze(0) == labels.unsqueeze(1)) & ~eye
        logp = sim - torch.logsumexp(sim, dim=1, keepdim=True)
        n_pos = pos.sum(1)
        loss = -(self.t / self.base_t) * (logp.masked_fill(~pos, 0).sum(1) / n_pos.clamp(min=1))
        if not (n_pos > 0).any():
            return sim.nan_to_num(neginf=0.0).sum() * 0
        return _reduce(loss[n_pos > 0], self.reduction)


# ------------------------------------------------------------------------------------------------ MoE auxiliary
class ZLoss(nn.Module):
    @reference_kwargs(z_loss_coef="weight")
    def __init__(self, weight: float = 1e-3):
        super().__init__()
        self.weight = weight

    def forward(self, router_logits):
        return self.weight * (torch.logsumexp(router_logits.float(), dim=-1) ** 2).mean()


class LoadBalancingLoss(nn.Module):
    """E * sum_i f_i P_i (f = fraction of tokens routed to expert i, P = mean router probability)."""

    @reference_kwargs(aux_loss_coef="weight")
    def __init__(self, num_experts: int, top_k: int = 1, weight: float = 1e-2):
        super().__init__()
        self.E, self.k, self.weight = num_experts, top_k, weight

    def forward(self, router_logits=None, expert_indices=None, *, router_probs=None):
        """From router LOGITS (soft-max taken here), or from probabilities via `router_probs=` (the reference's
        argument)."""
        probs = router_probs.float().reshape(-1, self.E) if router_probs is not None else \
            torch.softmax(router_logits.float().reshape(-1, self.E), -1)
        if expert_indices is None:
            expert_indices = probs.topk(self.k, dim=-1).indices
        f = F.one_hot(expert_indices.reshape(-1), self.E).float().mean(0) * 1.0
        return self.weight * self.E * (f * probs.mean(0)).sum()


class ExpertEntropyLoss(nn.Module):
    """Rewards high entropy of the AVERAGE expert usage (router logits in).  The reference's form
    `ExpertEntropyLoss(entropy_coef, target_entropy)(router_probs=...)` regularises the per-token routing entropy
    instead: coef * mean entropy, or coef * mean (entropy - target)^2."""

    @reference_kwargs(entropy_coef="weight")
    def __init__(self, weight: float = 1e-3, target_entropy: float | None = None):
        super().__init__()
        self.weight, self.target_entropy = weight, target_entropy

    def forward(self, router_logits=None, *, router_probs=None):
        if router_probs is not None:
            ent = -(router_probs.float() * (router_probs.float() + 1e-9).log()).sum(-1)
            return self.weight * ((ent - self.target_entropy).pow(2).mean() if self.target_entropy is not None else ent.mean())
        p = torch.softmax(router_logits.float(), -1).reshape(-1, router_logits.shape[-1]).mean(0)
        return -self.weight * -(p * (p + 1e-9).log()).sum()   # maximise usage entropy


# ------------------------------------------------------------------------------------------------ regression / ranking / segmentation
class MSELoss(nn.MSELoss): ...
class MAELoss(nn.L1Loss): ...
class HuberLoss(nn.HuberLoss):
    @reference_kwargs(pred="input")
    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return super().forward(input, target)
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
    def __init__(self, smooth: float = 1.0, reduction: str = "mean", square_denominator: bool = False):
        super().__init__()
        self.smooth, self.reduction, self.square = smooth, reduction, square_denominator

    @reference_kwargs(pred="logits")
    def forward(self, logits, target):
        p = torch.sigmoid(logits.float()).flatten(1)
        t = target.float().flatten(1)
        inter = (p * t).sum(1)
        den = (p * p).sum(1) + (t * t).sum(1) if self.square else p.sum(1) + t.sum(1)
        return _reduce(1 - (2 * inter + self.smooth) / (den + self.smooth), self.reduction)


class TverskyLoss(nn.Module):
    def __init__(self, alpha: float = 0.5, beta: float = 0.5, smooth: float = 1.0, reduction: str = "mean"):
        super().__init__()
        self.a, self.b, self.smooth, self.reduction = alpha, beta, smooth, reduction

    @reference_kwargs(pred="logits")
    def forward(self, logits, target):
        p, t = torch.sigmoid(logits.float()).flatten(1), target.float().flatten(1)
        tp, fp, fn = (p * t).sum(1), (p * (1 - t)).sum(1), ((1 - p) * t).sum(1)
        return _reduce(1 - (tp + self.smooth) / (tp + self.a * fp + self.b * fn + self.smooth), self.reduction)


class BCEWithLogitsLoss(nn.BCEWithLogitsLoss): ...


from .extra import (AttentionDistillationLoss, BoundaryLoss, CharbonnierLoss, FeatureDistillationLoss,  # noqa: E402
                    FocalTverskyLoss, GHMCLoss, IoULoss, LambdaRankLoss, ListMLELoss, LossOutput, PerceptualLoss,
                    create_label_smoothing_matrix)


# ------------------------------------------------------------------------------------------------ registry / composition
class LossRegistry:
    _losses: dict[str, Callable[..., nn.Module]] = {}

    @classmethod
    @reference_kwargs(loss_class="factory")
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

    def __init__(self, parts: Mapping[str, tuple] | None = None, *, losses: Mapping[str, tuple] | None = None,
                 normalize_weights: bool = False):
        """`parts`: {name: (loss, weight, argument names)}, fed from keyword arguments.  `losses` (the reference's
        form): {name: (loss, weight)} - every loss then receives the SAME positional / keyword arguments and the forward
        returns `LossOutput`; `normalize_weights` scales the weights to sum to 1."""
        super().__init__()
        self.broadcast = parts is None
        parts = dict(parts if parts is not None else {n: (m, w, ()) for n, (m, w) in (losses or {}).items()})
        self.names = list(parts)
        self.mods = nn.ModuleList(p[0] for p in parts.values())
        self.weights = [float(p[1]) for p in parts.values()]
        if normalize_weights and sum(self.weights) > 0:
            tot = sum(self.weights)
            self.weights = [w / tot for w in self.weights]
        self.args = [list(p[2]) for p in parts.values()]

    def forward(self, *args, **kw):
        if self.broadcast:
            total, metrics = 0.0, {}
            for n, m, w in zip(self.names, self.mods, self.weights):
                v = m(*args, **kw)
                v = v.loss if hasattr(v, "loss") else (v[0] if isinstance(v, tuple) else v)
                total = total + w * v
                metrics[f"{n}/loss"], metrics[f"{n}/weighted"] = v, w * v
            return _ref_output(total, total_loss=total, **metrics)
        total, detail = 0.0, {}
        for n, m, w, a in zip(self.names, self.mods, self.weights, self.args):
            v = m(*[kw[k] for k in a])
            v = v[0] if isinstance(v, tuple) else v
            detail[n] = v.detach()
            total = total + w * v
        return total, detail


class MultiTaskLoss(nn.Module):
    """Homoscedastic-uncertainty weighting: sum_i exp(-s_i) L_i + s_i."""

    def __init__(self, num_tasks: int | None = None, *, task_names: Sequence[str] | None = None,
                 loss_fns: Sequence[Callable] | None = None, learnable_weights: bool = True):
        """`MultiTaskLoss(n)` weights n ready loss values.  The reference's form names the tasks and their loss
        functions: `forward(predictions, targets)` (dicts keyed by task) then evaluates them itself, weights them as
        0.5 exp(-s_i) L_i + 0.5 s_i and returns `LossOutput`; `learnable_weights=False` freezes s_i = 0."""
        super().__init__()
        self.task_names = list(task_names) if task_names is not None else None
        self.loss_fns = nn.ModuleList(loss_fns) if loss_fns is not None and all(isinstance(f, nn.Module) for f in loss_fns) \
            else (list(loss_fns) if loss_fns is not None else None)
        n = num_tasks if num_tasks is not None else len(self.task_names)
        self.log_vars = nn.Parameter(torch.zeros(n), requires_grad=learnable_weights)

    def forward(self, losses=None, targets=None, *, predictions=None):
        if predictions is not None or isinstance(losses, Mapping):
            predictions = predictions if predictions is not None else losses
            total, metrics = 0.0, {}
            for i, name in enumerate(self.task_names):
                if name not in predictions or name not in targets:
                    continue
                v = self.loss_fns[i](predictions[name], targets[name])
                v = v.loss if hasattr(v, "loss") else v
                prec = torch.exp(-self.log_vars[i])
                total = total + 0.5 * prec * v + 0.5 * self.log_vars[i]
                metrics[f"{name}/loss"], metrics[f"{name}/weight"] = v, prec
            return _ref_output(total, total_loss=total, **metrics)
        return sum(torch.exp(-self.log_vars[i]) * l + self.log_vars[i] for i, l in enumerate(losses))


def create_loss(name="cross_entropy", **kw) -> nn.Module:
    """`create_loss("focal", gamma=2.0)`, or `create_loss(config)` with a loss configuration object (anything with a
    `type` field, e.g. the `loss` section of a SOTAConfig), as in data_pipeline/trainer/loss/__init__.py."""
    if hasattr(name, "type") and not isinstance(name, str):
        return create_loss_from_config(name)
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


# ---- constants and type aliases of data_pipeline/trainer/loss/sota_losses.py
from typing import Literal as _Literal  # noqa: E402

CACHE_LINE_BYTES, WARP_SIZE = 64, 32
MAX_VOCAB_CHUNK = 65536                    # widest vocabulary slice one pass of the chunked losses upcasts
EPS, LOG_MIN = 1e-8, -100.0
ReductionMode = _Literal["mean", "sum", "none", "batchmean"]
PreferenceLossType = _Literal["sigmoid", "hinge", "ipo", "kto", "robust"]


from ..config.sota_config import LossConfig as SOTALossConfig  # noqa: E402,F401  (alias of data_pipeline/trainer/loss/__init__.py)
