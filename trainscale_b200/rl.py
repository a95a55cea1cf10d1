"""RL / preference-training utilities and the preference trainer (DPO / SimPO / ORPO / KTO / CPO).

Utilities after data_pipeline/trainer/rl_training.py:95-671 (`selective_log_softmax`, `chunked_log_softmax`,
`compute_advantages` (group-normalised), `grpo_loss`, `drgrpo_loss`, `dapo_loss`, `left_pack_padding`, `GRPOCompute`,
`RewardModel`).  The reference ships the data stage and the losses but no preference training loop
(data_pipeline/trainer/loss/sota_losses.py:1151, preprocessing/prompt_engine.py:1929); `PreferenceTrainer` is that
loop: policy (and a frozen reference copy) under the flat engine, chosen and rejected sequences concatenated into
one forward, per-token log-probs from the fused lm_head + log-prob kernel (logits never materialised).
"""
from __future__ import annotations

import copy
from typing import Any, Dict

import torch
import torch.nn as nn
import torch.nn.functional as F

from .losses import CPOLoss, DPOLoss, KTOLoss, ORPOLoss, SimPOLoss
from .ops import cross_entropy as ce_ops
from .utils.refargs import ANY, reference_kwargs


@reference_kwargs(input_ids="index")
def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor, temperature: float = 1.0,
                          logit_softcapping: float = 0.0, logit_scale: float = 0.0) -> torch.Tensor:
    """log_softmax(logits)[..., index] without keeping the full log-softmax.  Optional transforms of the logits, in
    this order: soft-cap c tanh(z / c), scale, divide by the temperature."""
    if logit_softcapping:
        logits = logit_softcapping * torch.tanh(logits / logit_softcapping)
    if logit_scale:
        logits = logits * logit_scale
    if temperature != 1.0:
        logits = logits / temperature
    sel = logits.gather(-1, index.unsqueeze(-1)).squeeze(-1).float()
    return sel - torch.logsumexp(logits.float(), dim=-1)


@reference_kwargs(hidden_states="hidden", input_ids="labels")
def chunked_log_softmax(hidden: torch.Tensor, lm_head: torch.Tensor, labels: torch.Tensor, chunk_tokens: int = 4096,
                        ignore_index: int = -100, *, num_chunks: int | None = None, temperature: float = 1.0,
                        logit_softcapping: float = 0.0, logit_scale: float = 0.0) -> torch.Tensor:
    """Per-token log p(label) from hidden states, chunked over tokens: only [B, L] values are kept.  `num_chunks`
    (the reference's knob) sets the chunk size to tokens / num_chunks.  Temperature and logit scale act on the hidden
    states (the head is linear); soft-capping is not linear and takes the chunked PyTorch path."""
    tokens = labels.numel()
    if num_chunks:
        chunk_tokens = max(1, -(-tokens // int(num_chunks)))
    if logit_softcapping:
        h2, y = hidden.reshape(-1, hidden.shape[-1]), labels.reshape(-1)
        out = []
        for a in range(0, tokens, chunk_tokens):
            z = h2[a:a + chunk_tokens].float() @ lm_head.float().t()
            out.append(selective_log_softmax(z, y[a:a + chunk_tokens].clamp(min=0), temperature, logit_softcapping,
                                             logit_scale) * (y[a:a + chunk_tokens] != ignore_index))
        return torch.cat(out).view(labels.shape)
    factor = (logit_scale or 1.0) / temperature
    if factor != 1.0:
        hidden = hidden * factor
    return ce_ops.fused_linear_token_logprobs(hidden, lm_head, labels, ignore_index, chunk_tokens)


def compute_advantages(rewards: torch.Tensor, group_size: int | str | None = None, eps: float = 1e-4, scale: bool = True,
                       *, baseline: str | None = None) -> torch.Tensor:
    """Group-normalised advantages: rewards [N] with consecutive groups of `group_size` samples per prompt.

    The reference's form `compute_advantages(rewards [B, G], baseline="mean" | "max" | "min" | "none", eps)` subtracts the
    per-row baseline and divides by the standard deviation of ALL advantages (data_pipeline/trainer/rl_training.py:241);
    it is selected by `baseline=` or by a string in the second position, and returns the [B, G] shape."""
    if isinstance(group_size, str) or baseline is not None or group_size is None:
        kind = baseline if baseline is not None else (group_size or "mean")
        r = rewards.float()
        base = {"mean": lambda: r.mean(-1, keepdim=True), "max": lambda: r.max(-1, keepdim=True).values,
                "min": lambda: r.min(-1, keepdim=True).values}.get(kind, lambda: 0.0)()
        a = r - base
        std = a.std() if a.numel() > 1 else a.new_zeros(())
        return a / std if float(std) > eps else a
    r = rewards.float().view(-1, group_size)
    a = r - r.mean(1, keepdim=True)
    if scale:
        a = a / (r.std(1, keepdim=True) + eps)
    return a.reshape(-1)


def _masked_mean(x, mask, dim=None):
    return (x * mask).sum(dim) / mask.sum(dim).clamp(min=1)


def _seq_mean(x, mask):
    return (x * mask).sum(-1) / mask.sum(-1).clamp(min=1)


def _reference_rl_loss(kind: str, policy_log_probs, ref_log_probs, third, mask, beta=0.04, epsilon=0.1, temperature=1.0):
    """The reference's sequence-level formulations (data_pipeline/trainer/rl_training.py:297-430), returning
    (loss, metrics).  grpo: -E[A * mean log pi] + beta * KL-per-token; drgrpo: PPO-style clipping of the sequence-level
    ratio pi / pi_ref; dapo: policy gradient weighted by softmax(rewards / temperature) over each group."""
    lp, lr = _seq_mean(policy_log_probs, mask), _seq_mean(ref_log_probs, mask)
    log_ratio = policy_log_probs - ref_log_probs
    metrics = {}
    if kind == "grpo":
        pg = -(third * lp).mean()
        kl_tok = log_ratio * mask
        kl = beta * kl_tok.sum(-1).mean() / mask.sum(-1).clamp(min=1).mean()
        metrics["kl_div"] = float((kl_tok.mean()).detach())
    elif kind == "drgrpo":
        ratio = torch.exp(_seq_mean(log_ratio, mask))
        adv = third.reshape(-1)
        pg = -torch.minimum(ratio.reshape(-1) * adv, ratio.clamp(1 - epsilon, 1 + epsilon).reshape(-1) * adv).mean()
        kl_seq = _seq_mean(log_ratio, mask)
        kl = beta * kl_seq.mean()
        metrics.update(kl_div=float((kl_seq.mean()).detach()), ratio_mean=float((ratio.mean()).detach()))
    else:
        soft = torch.softmax(third.float() / temperature, dim=-1)
        pg = -(soft * lp).sum(-1).mean()
        kl = beta * _seq_mean(log_ratio, mask).mean()
        metrics["soft_advantages_entropy"] = float(-(soft * soft.clamp_min(1e-30).log()).sum(-1).mean().detach())
    loss = pg + kl
    metrics.update(pg_loss=float((pg).detach()), kl_loss=float((kl).detach()), total_loss=float((loss).detach()))
    return loss, metrics


def grpo_loss(logp: torch.Tensor = None, old_logp: torch.Tensor = None, ref_logp: torch.Tensor | None = None,
              advantages: torch.Tensor = None, mask: torch.Tensor = None, clip: float = 0.2, beta: float = 0.01, *,
              policy_log_probs=None, ref_log_probs=None):
    """Clipped surrogate per token, averaged per sequence then over the batch, plus the k3 KL estimator.
    Called with the reference's keywords (`policy_log_probs=, ref_log_probs=, advantages=, mask=, beta=`) it computes
    the reference's sequence-level loss instead and returns (loss, metrics): see `_reference_rl_loss`."""
    if policy_log_probs is not None:
        return _reference_rl_loss("grpo", policy_log_probs, ref_log_probs, advantages, mask, beta)
    ratio = torch.exp(logp - old_logp)
    a = advantages.unsqueeze(-1)
    obj = torch.minimum(ratio * a, ratio.clamp(1 - clip, 1 + clip) * a)
    per_tok = -obj
    if ref_logp is not None and beta > 0:
        d = ref_logp - logp
        per_tok = per_tok + beta * (torch.exp(d) - d - 1)
    return _masked_mean(per_tok, mask, dim=-1).mean()


def drgrpo_loss(logp=None, old_logp=None, advantages=None, mask=None, clip: float = 0.2, max_len: int | None = None, *,
                policy_log_probs=None, ref_log_probs=None, beta: float = 0.04, epsilon: float = 0.1):
    """Dr. GRPO: no std scaling in the advantage and a constant length normaliser (removes the length bias).
    With the reference's keywords (`policy_log_probs=, ref_log_probs=, ..., beta=, epsilon=`): its formulation,
    returning (loss, metrics)."""
    if policy_log_probs is not None:
        return _reference_rl_loss("drgrpo", policy_log_probs, ref_log_probs, advantages, mask, beta, epsilon)
    ratio = torch.exp(logp - old_logp)
    a = advantages.unsqueeze(-1)
    obj = torch.minimum(ratio * a, ratio.clamp(1 - clip, 1 + clip) * a)
    L = max_len or mask.shape[-1]
    return -((obj * mask).sum(-1) / L).mean()


def dapo_loss(logp=None, old_logp=None, advantages=None, mask=None, clip_low: float = 0.2, clip_high: float = 0.28, *,
              policy_log_probs=None, ref_log_probs=None, rewards=None, beta: float = 0.04, temperature: float = 1.0):
    """DAPO: decoupled clip range and token-level normalisation over the whole batch.  With the reference's keywords
    (`policy_log_probs=, ref_log_probs=, rewards=, mask=, beta=, temperature=`): its soft-advantage formulation,
    returning (loss, metrics)."""
    if policy_log_probs is not None:
        return _reference_rl_loss("dapo", policy_log_probs, ref_log_probs, rewards, mask, beta, temperature=temperature)
    ratio = torch.exp(logp - old_logp)
    a = advantages.unsqueeze(-1)
    obj = torch.minimum(ratio * a, ratio.clamp(1 - clip_low, 1 + clip_high) * a)
    return -(obj * mask).sum() / mask.sum().clamp(min=1)


@reference_kwargs(input_ids="ids")
def left_pack_padding(ids: torch.Tensor, mask: torch.Tensor | int | None = None, pad_id: int = 0, *,
                      pad_token_id: int | None = None):
    """Move real tokens to the left of every row (stable), padding to the right: returns (ids, mask).

    The reference's function of this name, `left_pack_padding(input_ids, pad_token_id)`, goes the other way: it moves
    the PADDING to the left (real tokens end flush right, as its attention path wants) and returns the ids alone
    (data_pipeline/trainer/rl_training.py:434).  That form is selected by an integer second argument or `pad_token_id=`."""
    if pad_token_id is not None or isinstance(mask, int):
        pad = pad_token_id if pad_token_id is not None else mask
        real = ids != pad
        order = torch.argsort(real.int(), dim=1, stable=True)          # padding first, tokens keep their order
        return ids.gather(1, order)
    order = torch.argsort((mask == 0).int(), dim=1, stable=True)
    return ids.gather(1, order).masked_fill(mask.gather(1, order) == 0, pad_id), mask.gather(1, order)


class GRPOCompute:
    def __init__(self, group_size: int = 8, clip: float = 0.2, beta: float = 0.01, variant: str = "grpo",
                 model: nn.Module | None = None, reward_clip: float | None = None, chunk_tokens: int = 4096, *,
                 ref_model: nn.Module | None = None, config=None):
        """`GRPOCompute(model, ref_model, config)` is the reference's form: `config` (an RL configuration object)
        supplies num_generations (group size), clip_range, kl_coef (beta), algorithm (variant) and reward_clip."""
        if isinstance(group_size, nn.Module):                 # positional (model, ref_model, config)
            model, group_size = group_size, 8
            if isinstance(clip, nn.Module) or clip is None:
                ref_model, clip = clip, 0.2
            if not isinstance(beta, (int, float)):
                config, beta = beta, 0.01
        if config is not None:
            group_size = int(getattr(config, "num_generations", group_size))
            clip = float(getattr(config, "clip_range", clip))
            beta = float(getattr(config, "kl_coef", beta))
            variant = str(getattr(getattr(config, "algorithm", variant), "value", getattr(config, "algorithm", variant))).lower()
            reward_clip = getattr(config, "reward_clip", reward_clip)
        self.group_size, self.clip, self.beta, self.variant = group_size, clip, beta, variant
        self.model, self.ref_model, self.reward_clip, self.chunk_tokens = model, ref_model, reward_clip, chunk_tokens

    def compute_log_probs(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None,
                          model: nn.Module | None = None) -> torch.Tensor:
        """log p(token t+1 | tokens <= t) for every position, [B, S-1] (0 where the target is padding), without ever
        forming [B, S, V] logits: the decoder's hidden states go through the chunked fused head
        (data_pipeline/trainer/rl_training.py:509-552)."""
        model = model if model is not None else self.model
        if model is None:
            raise ValueError("compute_log_probs needs a model (argument or constructor)")
        out = model(input_ids=input_ids, return_logits=False)
        labels = input_ids[:, 1:]
        if attention_mask is not None:
            labels = labels.masked_fill(attention_mask[:, 1:] == 0, -100)
        return chunked_log_softmax(out.hidden_states[:, :-1], model.head_weight, labels, self.chunk_tokens)

    def compute_grpo_loss(self, policy_log_probs, ref_log_probs, rewards, mask, old_log_probs=None):
        """(loss, {"reward_mean", "reward_std", "advantage_abs_mean", "kl"}) for the configured variant.  Without
        `old_log_probs` the policy's own (detached) values are the behaviour policy: one optimisation step per batch."""
        if self.reward_clip:
            rewards = rewards.clamp(-self.reward_clip, self.reward_clip)
        old = policy_log_probs.detach() if old_log_probs is None else old_log_probs
        loss = self(policy_log_probs, old, ref_log_probs, rewards, mask)
        adv = compute_advantages(rewards, self.group_size, scale=self.variant != "drgrpo")
        stats = {"reward_mean": float(rewards.float().mean()), "reward_std": float(rewards.float().std()),
                 "advantage_abs_mean": float(adv.abs().mean())}
        if ref_log_probs is not None:
            d = (ref_log_probs - policy_log_probs).detach()
            stats["kl"] = float(_masked_mean(torch.exp(d) - d - 1, mask))
        return loss, stats

    def __call__(self, logp, old_logp, ref_logp, rewards, mask):
        adv = compute_advantages(rewards, self.group_size, scale=self.variant != "drgrpo")
        if self.variant == "drgrpo":
            return drgrpo_loss(logp, old_logp, adv, mask, self.clip)
        if self.variant == "dapo":
            return dapo_loss(logp, old_logp, adv, mask, self.clip)
        return grpo_loss(logp, old_logp, ref_logp, adv, mask, self.clip, self.beta)


class RewardModel(nn.Module):
    """Decoder backbone + scalar head read at the last real token."""

    def __init__(self, backbone=None, *, model=None, reward_fn=None):
        """`RewardModel(backbone)`: a framework decoder gets a scalar value head.  `model=` / `reward_fn=` are the
        reference's form (data_pipeline/trainer/rl_training.py:607): any classifier whose last-position logit is the
        score, or a function (input_ids, attention_mask, **kw) -> [B]; with neither, rewards are zero."""
        super().__init__()
        self.reward_fn, self.scorer = reward_fn, None
        backbone = backbone if backbone is not None else model
        self.backbone = backbone
        if backbone is not None and hasattr(getattr(backbone, "config", None), "hidden_size") and hasattr(backbone, "model"):
            h = backbone.config.hidden_size
            p = next(backbone.parameters())
            self.value_head = nn.Linear(h, 1, bias=False, dtype=p.dtype, device=p.device)
        else:
            self.scorer, self.backbone = backbone, None

    def forward(self, input_ids, attention_mask=None, **kwargs):
        if self.backbone is None:
            if self.scorer is not None:
                out = self.scorer(input_ids=input_ids, attention_mask=attention_mask)
                logits = out.logits if hasattr(out, "logits") else out
                return logits[:, -1].reshape(logits.shape[0], -1)[:, 0].float() if logits.dim() > 1 else logits.float()
            if self.reward_fn is not None:
                return self.reward_fn(input_ids, attention_mask, **kwargs)
            return torch.zeros(input_ids.shape[0], device=input_ids.device)
        h = self.backbone.model(input_ids)
        if attention_mask is None:
            last = torch.full((h.shape[0],), h.shape[1] - 1, device=h.device)
        else:
            last = attention_mask.long().sum(1).clamp(min=1) - 1
        return self.value_head(h[torch.arange(h.shape[0], device=h.device), last]).squeeze(-1).float()


class PreferenceTrainer:
    """Preference optimisation on batches with chosen_/rejected_ input_ids, attention_mask and labels."""

    def __init__(self, policy, engine=None, ref_model=None, loss: str = "dpo", beta: float = 0.1, **loss_kw):
        self.policy, self.engine, self.kind = policy, engine, loss
        self.ref = ref_model
        if self.ref is not None:
            self.ref.eval()
            for p in self.ref.parameters():
                p.requires_grad_(False)
        self.loss_fn = {"dpo": lambda: DPOLoss(beta, **loss_kw), "simpo": lambda: SimPOLoss(beta, **loss_kw),
                        "orpo": lambda: ORPOLoss(**loss_kw), "kto": lambda: KTOLoss(beta, **loss_kw),
                        "cpo": lambda: CPOLoss(beta, **loss_kw)}[loss]()

    @staticmethod
    def make_reference(policy):
        """Frozen copy of the policy taken before the engine re-points its parameters at flat buffers."""
        ref = copy.deepcopy(policy)
        for p in ref.parameters():
            p.requires_grad_(False)
        return ref.eval()

    def _seq_logps(self, model, ids, mask, labels, grad: bool):
        ctx = torch.enable_grad() if grad else torch.no_grad()
        with ctx:
            h = model.model(ids)
            w = model.head_weight
            lab = labels.masked_fill(mask == 0, -100)
            tgt = torch.full_like(lab, -100)
            tgt[:, :-1] = lab[:, 1:]
            lp = ce_ops.fused_linear_token_logprobs(h, w if grad else w.detach(), tgt)
            return lp.sum(-1), (tgt != -100).sum(-1)

    def compute_loss(self, batch: Dict[str, torch.Tensor]):
        B = batch["chosen_input_ids"].shape[0]
        ids = torch.cat((batch["chosen_input_ids"], batch["rejected_input_ids"]))
        mask = torch.cat((batch["chosen_attention_mask"], batch["rejected_attention_mask"]))
        labels = torch.cat((batch["chosen_labels"], batch["rejected_labels"]))
        lp, n = self._seq_logps(self.policy, ids, mask, labels, True)
        pc, pr, nc, nr = lp[:B], lp[B:], n[:B], n[B:]
        metrics = {}
        if self.kind == "dpo":
            rc = rr = None
            if self.ref is not None and not self.loss_fn.reference_free:
                rl, _ = self._seq_logps(self.ref, ids, mask, labels, False)
                rc, rr = rl[:B], rl[B:]
            loss, cr, rjr = self.loss_fn(pc, pr, rc, rr)
            metrics = {"reward_accuracy": (cr > rjr).float().mean(), "reward_margin": (cr - rjr).mean()}
        elif self.kind == "simpo":
            loss, cr, rjr = self.loss_fn(pc, pr, nc.float(), nr.float())
            metrics = {"reward_accuracy": (cr > rjr).float().mean()}
        elif self.kind == "orpo":
            nll = -(pc / nc.clamp(min=1)).mean()
            loss, ratio = self.loss_fn(pc / nc.clamp(min=1), pr / nr.clamp(min=1), nll)
            metrics = {"log_odds_ratio": ratio.mean()}
        elif self.kind == "cpo":
            loss = self.loss_fn(pc, pr, -(pc / nc.clamp(min=1)).mean())
        else:   # kto on paired data: chosen = desirable, rejected = undesirable
            rl = torch.zeros_like(lp)
            if self.ref is not None:
                rl, _ = self._seq_logps(self.ref, ids, mask, labels, False)
            tag = torch.cat((torch.ones(B), torch.zeros(B))).to(lp.device)
            loss, _ = self.loss_fn(lp, rl, tag)
        return loss, metrics

    def train_step(self, batch: Dict[str, torch.Tensor], lr: float | None = None):
        loss, metrics = self.compute_loss(batch)
        if self.engine is not None:
            self.engine.micro_step = max(1, self.engine.cfg.gradient_accumulation_steps) - 1
            self.engine.backward(loss)
            gn = self.engine.step(lr)
        else:
            loss.backward()
            gn = None
        return loss.detach(), metrics, gn


# ------------------------------------------------------------------------------------------------ reward / batch helpers
def clip_rewards(rewards: torch.Tensor, clip_value: float | None = 10.0) -> torch.Tensor:
    """Clamp rewards to [-clip_value, clip_value] (data_pipeline/trainer/rl_training.py:272)."""
    return rewards if clip_value is None else rewards.clamp(-clip_value, clip_value)


def apply_length_penalty(rewards: torch.Tensor, lengths: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """rewards * (length / longest length)^alpha: short completions earn less (rl_training.py:282)."""
    return rewards * (lengths.float() / lengths.max().clamp(min=1).float()) ** alpha


def calculate_pad_tokens_in_prompt(input_ids: torch.Tensor, logits_to_keep: int, pad_token_id: int) -> torch.Tensor:
    """Pad tokens in the prompt part (everything but the last `logits_to_keep` positions) of every row."""
    return (input_ids[:, :-logits_to_keep] == pad_token_id).sum(-1)


def create_completion_attention_mask(input_ids: torch.Tensor, pad_token_id: int) -> torch.Tensor:
    return (input_ids != pad_token_id).long()


def autotune_batch_and_chunks(total_rows: int, seq_len: int, hidden_dim: int, vocab_dim: int, dtype_bytes: int = 16,
                              multiplier: int | None = None, budget_bytes: int | None = None) -> tuple[int, int]:
    """(rows per pass, number of vocabulary chunks) for a chunked log-softmax over `total_rows` sequences
    (rl_training.py:198-238).  A pass holds rows x seq_len hidden states and one chunk of the logits, rows x seq_len x
    vocab / chunks in fp32; rows is the largest divisor of `total_rows` that fits the budget (default 4 GiB; on a
    180 GB part pass `budget_bytes`), chunks defaults to max(4, seq_len / 4096).  `dtype_bytes` is in BITS, as in the
    reference."""
    chunks = multiplier if multiplier is not None else max(4, seq_len // 4096)
    budget = budget_bytes if budget_bytes is not None else 4 * 2 ** 30
    per_row = seq_len * hidden_dim * dtype_bytes / 8 + seq_len * vocab_dim * 4 / chunks
    rows = int(max(1, min(total_rows, budget // max(per_row, 1))))
    while total_rows % rows:
        rows -= 1
    return rows, chunks


# ---- the three group-relative losses in the reference's POSITIONAL order (data_pipeline/trainer/rl_training.py:297-440):
# what `from data_pipeline.trainer.rl_training import grpo_loss` resolves to under `reference_paths`, so that
# `grpo_loss(policy_log_probs, ref_log_probs, advantages, mask, beta)` called by position means what it means there
def _reference_grpo_loss(policy_log_probs, ref_log_probs, advantages, mask, beta: float = 0.04):
    return grpo_loss(policy_log_probs=policy_log_probs, ref_log_probs=ref_log_probs, advantages=advantages, mask=mask,
                     beta=beta)


def _reference_drgrpo_loss(policy_log_probs, ref_log_probs, advantages, mask, beta: float = 0.04, epsilon: float = 0.1):
    return drgrpo_loss(policy_log_probs=policy_log_probs, ref_log_probs=ref_log_probs, advantages=advantages, mask=mask,
                       beta=beta, epsilon=epsilon)


def _reference_dapo_loss(policy_log_probs, ref_log_probs, rewards, mask, beta: float = 0.04, temperature: float = 1.0):
    return dapo_loss(policy_log_probs=policy_log_probs, ref_log_probs=ref_log_probs, rewards=rewards, mask=mask, beta=beta,
                     temperature=temperature)


grpo_loss.__reference_form__ = _reference_grpo_loss
drgrpo_loss.__reference_form__ = _reference_drgrpo_loss
dapo_loss.__reference_form__ = _reference_dapo_loss
