"""Speculative decoding (draft-and-verify) and multi-adapter LoRA serving.

Speculative decoding: a small draft model proposes `k` tokens one at a time, the target model scores all of them in ONE
forward over `k + 1` positions, and the standard accept / resample rule keeps the output distribution exactly the
target's (for greedy decoding: exactly the target's greedy continuation).  The reference only configures this in vLLM
(data_pipeline/trainer/inference.py:786-921, `SpeculativeConfig`); here it runs on the framework's own decoder with a
dense per-layer KV cache that can be rolled back to the accepted length.

Multi-LoRA serving: `LoRAAdapterRegistry` keeps several adapters' low-rank weights for one attached set of LoRA
modules and switches between them per request group (`LoRAServingConfig.max_loras`).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ops.attention import _split_qkv, attention_reference


class DenseKVCache:
    """One layer's K/V for a single sequence: [1, max_len, Hkv, D].  `seq_len` is advanced by the caller after the
    whole forward (every layer must see the same offset) and can be moved back to drop rejected tokens."""

    def __init__(self, max_len: int, n_kv: int, head_dim: int, dtype, device):
        self.k = torch.zeros(1, max_len, n_kv, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.seq_len = 0

    def attend(self, qkv: torch.Tensor, attn) -> torch.Tensor:
        B, S, _ = qkv.shape
        q, k, v = _split_qkv(qkv, attn.n_heads, attn.n_kv, attn.hd)
        a, b = self.seq_len, self.seq_len + S
        self.k[:, a:b] = k
        self.v[:, a:b] = v
        o = attention_reference(q, self.k[:, :b], self.v[:, :b], True, None, attn.cfg.sliding_window,
                                attn.cfg.attn_logit_softcap)
        return o.reshape(B, S, attn.n_heads * attn.hd)


def make_caches(model, max_len: int) -> list[DenseKVCache]:
    cfg = model.config
    p = next(model.parameters())
    return [DenseKVCache(max_len, cfg.num_key_value_heads, cfg.head_dim, p.dtype, p.device)
            for _ in range(cfg.num_hidden_layers)]


@torch.no_grad()
def _forward(model, ids: torch.Tensor, caches: list[DenseKVCache]) -> torch.Tensor:
    """Logits [S, V] (fp32) of `ids` [S] appended to the cached prefix; advances the caches."""
    h = model.model(ids.view(1, -1), kv_caches=caches)
    for c in caches:
        c.seq_len += ids.numel()
    return model.logits(h)[0].float()


def _set_len(caches: list[DenseKVCache], n: int) -> None:
    for c in caches:
        c.seq_len = n


def _probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    return torch.softmax(logits / max(temperature, 1e-6), dim=-1)


@dataclass
class SpeculativeStats:
    proposed: int = 0
    accepted: int = 0
    target_forwards: int = 0
    per_round: list = field(default_factory=list)

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / max(1, self.proposed)


@torch.no_grad()
def speculative_generate(target, draft, prompt_ids: list[int], max_new_tokens: int, k: int = 4,
                         temperature: float = 0.0, eos_token_id: int | None = None,
                         generator: torch.Generator | None = None) -> tuple[list[int], SpeculativeStats]:
    """Returns (generated token ids, statistics).  temperature == 0: greedy, output identical to the target's own
    greedy decode.  temperature > 0: rejection sampling, output distributed exactly as sampling from the target."""
    dev = next(target.parameters()).device
    n_ctx = len(prompt_ids) + max_new_tokens + k + 2
    tc, dc = make_caches(target, n_ctx), make_caches(draft, n_ctx)
    ids = torch.tensor(prompt_ids, dtype=torch.long, device=dev)
    stats = SpeculativeStats()
    # prefill both models on the prompt; `t_last` is the target's distribution for the next token
    t_last = _forward(target, ids, tc)[-1]
    stats.target_forwards += 1
    d_last = _forward(draft, ids, dc)[-1]
    out: list[int] = []
    greedy = temperature <= 0.0

    def pick(p_or_logits):
        if greedy:
            return int(torch.argmax(p_or_logits))
        return int(torch.multinomial(p_or_logits, 1, generator=generator))

    # first token comes straight from the target's prefill
    nxt = pick(t_last if greedy else _probs(t_last, temperature))
    out.append(nxt)
    while len(out) < max_new_tokens and nxt != eos_token_id:
        base_t, base_d = tc[0].seq_len, dc[0].seq_len
        # the draft continues from `nxt` for k steps
        proposals, q_dists = [], []
        cur = nxt
        for _ in range(k):
            dl = _forward(draft, torch.tensor([cur], device=dev), dc)[-1]
            q = dl if greedy else _probs(dl, temperature)
            cur = pick(q)
            proposals.append(cur)
            q_dists.append(q)
        # the target scores [nxt, d1 .. dk] in one forward: row i is its distribution after the i-th of them
        tl = _forward(target, torch.tensor([nxt] + proposals, device=dev), tc)
        stats.target_forwards += 1
        stats.proposed += k
        n_acc = 0
        replacement = None
        for i, d in enumerate(proposals):
            if greedy:
                best = int(torch.argmax(tl[i]))
                if best == d:
                    n_acc += 1
                    continue
                replacement = best
                break
            p, q = _probs(tl[i], temperature), q_dists[i]
            u = torch.rand((), generator=generator, device=p.device if generator is None else generator.device).to(p.device)
            if u <= torch.clamp(p[d] / q[d].clamp(min=1e-20), max=1.0):
                n_acc += 1
                continue
            resid = torch.clamp(p - q, min=0.0)
            replacement = pick(resid / resid.sum().clamp(min=1e-20))
            break
        stats.accepted += n_acc
        stats.per_round.append(n_acc)
        accepted = proposals[:n_acc]
        if replacement is None:     # everything accepted: one bonus token from the target's last row
            replacement = pick(tl[k] if greedy else _probs(tl[k], temperature))
        new_tokens = accepted + [replacement]
        for tkn in new_tokens:
            out.append(tkn)
            if tkn == eos_token_id or len(out) >= max_new_tokens:
                break
        nxt = out[-1]
        # keep [nxt_old, accepted...] in both caches; the replacement token is fed at the next round
        _set_len(tc, base_t + 1 + n_acc)
        _set_len(dc, min(base_d + 1 + n_acc, dc[0].seq_len))
        if dc[0].seq_len < base_d + 1 + n_acc:
            # all k proposals accepted: the draft has not seen its own last proposal yet
            _forward(draft, torch.tensor([accepted[-1]], device=dev), dc)
    return out[:max_new_tokens], stats


@torch.no_grad()
def greedy_generate(model, prompt_ids: list[int], max_new_tokens: int, eos_token_id: int | None = None) -> list[int]:
    """Plain cached greedy decode (the oracle for the speculative path)."""
    dev = next(model.parameters()).device
    caches = make_caches(model, len(prompt_ids) + max_new_tokens + 1)
    logits = _forward(model, torch.tensor(prompt_ids, dtype=torch.long, device=dev), caches)[-1]
    out = []
    for _ in range(max_new_tokens):
        t = int(torch.argmax(logits))
        out.append(t)
        if t == eos_token_id:
            break
        logits = _forward(model, torch.tensor([t], device=dev), caches)[-1]
    return out


class LoRAAdapterRegistry:
    """Several named adapters for one model whose LoRA modules are already attached (`lora.get_peft_model`).
    `activate(name)` copies that adapter's low-rank weights into the attached modules; requests are grouped by adapter
    so that a switch happens once per group, and at most `max_loras` adapters stay resident on the device."""

    def __init__(self, model, max_loras: int = 4):
        self.model, self.max_loras = model, max_loras
        self._get = lambda: {n: p for n, p in model.named_parameters() if "lora_" in n}   # live tensors
        self.adapters: dict[str, dict[str, torch.Tensor]] = {}
        self._lru: list[str] = []
        self.active: str | None = None
        self.switches = 0

    def register(self, name: str, state: dict[str, torch.Tensor] | None = None) -> None:
        """Store `state` (or a snapshot of the currently attached weights) under `name`."""
        src = state if state is not None else self._get()
        missing = set(self._get()) - set(src)
        if missing:
            raise KeyError(f"adapter {name!r} lacks {sorted(missing)[:3]}...")
        self.adapters[name] = {k: v.detach().clone() for k, v in src.items()}
        self._touch(name)

    def _touch(self, name: str) -> None:
        if name in self._lru:
            self._lru.remove(name)
        self._lru.append(name)
        while len(self._lru) > self.max_loras:
            victim = self._lru.pop(0)
            self.adapters[victim] = {k: v.cpu() for k, v in self.adapters[victim].items()}   # offloaded, not dropped

    @torch.no_grad()
    def activate(self, name: str | None) -> None:
        if name == self.active:
            return
        live = self._get()
        if name is None:
            for k, v in live.items():
                if k.endswith("lora_B"):
                    v.zero_()                    # zero B: the adapters contribute nothing
        else:
            st = self.adapters[name]
            for k, v in live.items():
                v.copy_(st[k].to(v.device))
            self._touch(name)
        self.active = name
        self.switches += 1

    def group_requests(self, adapter_of_request: list[str | None]) -> list[tuple[str | None, list[int]]]:
        """Request indices grouped by adapter, current adapter first (fewest switches)."""
        groups: dict[str | None, list[int]] = {}
        for i, a in enumerate(adapter_of_request):
            groups.setdefault(a, []).append(i)
        order = sorted(groups, key=lambda a: (a != self.active, str(a)))
        return [(a, groups[a]) for a in order]
