"""Token sampling: temperature, top-k, top-p, min-p, repetition / presence / frequency penalties, per-request seeds."""
from __future__ import annotations

import torch


def apply_penalties(logits: torch.Tensor, prev_tokens: list[list[int]], repetition: list[float], presence: list[float],
                    frequency: list[float]) -> torch.Tensor:
    for i, toks in enumerate(prev_tokens):
        if not toks or (repetition[i] == 1.0 and presence[i] == 0.0 and frequency[i] == 0.0):
            continue
        t = torch.tensor(toks, device=logits.device)
        uniq, counts = torch.unique(t, return_counts=True)
        row = logits[i]
        if repetition[i] != 1.0:
            v = row[uniq]
            row[uniq] = torch.where(v > 0, v / repetition[i], v * repetition[i])
        if presence[i] != 0.0:
            row[uniq] -= presence[i]
        if frequency[i] != 0.0:
            row[uniq] -= frequency[i] * counts.to(row.dtype)
    return logits


def sample(logits: torch.Tensor, temperature: list[float], top_k: list[int], top_p: list[float], min_p: list[float],
           generators: list[torch.Generator | None]) -> tuple[torch.Tensor, torch.Tensor]:
    """logits [B, V] fp32 -> (token ids [B], log-prob of the chosen token [B])."""
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.long, device=logits.device)
    logp_all = torch.log_softmax(logits, dim=-1)
    for i in range(B):
        row = logits[i]
        if temperature[i] <= 1e-5:
            out[i] = row.argmax()
            continue
        row = row / temperature[i]
        if top_k[i] and 0 < top_k[i] < V:
            kth = torch.topk(row, top_k[i]).values[-1]
            row = row.masked_fill(row < kth, float("-inf"))
        probs = torch.softmax(row, dim=-1)
        if min_p[i] and min_p[i] > 0:
            probs = probs.masked_fill(probs < min_p[i] * probs.max(), 0.0)
        if top_p[i] and top_p[i] < 1.0:
            sp, si = torch.sort(probs, descending=True)
            cum = torch.cumsum(sp, 0)
            cut = cum - sp > top_p[i]
            sp = sp.masked_fill(cut, 0.0)
            probs = torch.zeros_like(probs).scatter(0, si, sp)
        probs = probs / probs.sum().clamp(min=1e-20)
        g = generators[i]
        if g is not None and g.device != probs.device:
            out[i] = torch.multinomial(probs.cpu(), 1, generator=g).to(logits.device)[0]
        else:
            out[i] = torch.multinomial(probs, 1, generator=g)[0]
    return out, logp_all.gather(1, out.unsqueeze(1)).squeeze(1)
