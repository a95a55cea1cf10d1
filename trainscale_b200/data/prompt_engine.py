"""Prompt engine: raw dataset rows -> token tensors for pre-training, fine-tuning and preference / RL stages.

Output containers and stage behaviour follow data_pipeline/preprocessing/prompt_engine.py:118-2978:
  pre-training   causal LM, fill-in-the-middle (PSM / SPM, :872-936), T5-style span corruption (:940-1038),
                 document packing greedy / first-fit-decreasing with per-document position_ids and document_ids,
                 pad document_id = -1 (:1042-1228)
  fine-tuning    chat (prompt prefix masked up to the last assistant turn, :1300-1357), completion, instruction
                 (Alpaca-style), multi-turn (labels by role ranges, :1463-1546), custom template
  post-training  DPO / ORPO pairs ((prompt+response)[:max_len] padded to max_len, prompt labels masked,
                 :1896-1979), PPO prompts, KTO (tag + weight), GRPO groups with scores, reward-model pairs
Labels use -100 for ignored positions and are NOT shifted (the model shifts).
"""
from __future__ import annotations

import random
import re
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Mapping, Sequence

import torch

from ..config.data_schema import (FIMMode, FineTuningFormat, PackingConfig, PackingStrategy, PreTrainingFormat,
                                  PromptEngineConfig, PromptTemplate, RLAlgorithm, TrainingStage)
from ..core.errors import PipelineError, TemplateRenderError, TokenizationError
from ..utils.refargs import ANY, reference_kwargs
from .tokenization import TokenizerWrapper

IGNORE = -100


# ------------------------------------------------------------------------------------------------ containers
@dataclass
class ProcessedExample:
    input_ids: list[int]
    attention_mask: list[int]
    labels: list[int]
    extras: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        return {"input_ids": self.input_ids, "attention_mask": self.attention_mask, "labels": self.labels, **self.extras}


@dataclass
class PackedExample:
    input_ids: list[int]
    attention_mask: list[int]
    labels: list[int]
    position_ids: list[int]
    document_ids: list[int]
    num_documents: int
    cu_seqlens: list[int] = field(default_factory=list)

    def to_dict(self) -> dict:
        d = {"input_ids": self.input_ids, "attention_mask": self.attention_mask, "labels": self.labels,
             "position_ids": self.position_ids, "document_ids": self.document_ids, "num_documents": self.num_documents}
        if self.cu_seqlens:
            d["cu_seqlens"] = self.cu_seqlens
        return d


@dataclass
class PreferencePairExample:
    prompt_input_ids: list[int]
    prompt_attention_mask: list[int]
    chosen_input_ids: list[int]
    chosen_attention_mask: list[int]
    chosen_labels: list[int]
    rejected_input_ids: list[int]
    rejected_attention_mask: list[int]
    rejected_labels: list[int]

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass
class PPOExample:
    query_input_ids: list[int]
    query_attention_mask: list[int]
    query_text: str = ""

    def to_dict(self) -> dict:
        return {"input_ids": self.query_input_ids, "attention_mask": self.query_attention_mask,
                "query_input_ids": self.query_input_ids, "query_attention_mask": self.query_attention_mask}


@dataclass
class KTOExample:
    input_ids: list[int]
    attention_mask: list[int]
    labels: list[int]
    kto_tag: bool
    weight: float = 1.0

    def to_dict(self) -> dict:
        return {"input_ids": self.input_ids, "attention_mask": self.attention_mask, "labels": self.labels,
                "kto_tag": int(self.kto_tag), "weight": self.weight}


@dataclass
class GRPOExample:
    prompt_input_ids: list[int]
    prompt_attention_mask: list[int]
    responses_input_ids: list[list[int]]
    responses_attention_mask: list[list[int]]
    responses_labels: list[list[int]]
    scores: list[float]

    def to_dict(self) -> dict:
        return dict(self.__dict__)


# ------------------------------------------------------------------------------------------------ templates / labels
_VAR = re.compile(r"\{([A-Za-z_][A-Za-z0-9_]*)\}")


def render_template(template: str, variables: Mapping[str, Any], use_jinja: bool | None = None) -> str:
    """Jinja2 when the template uses `{{` / `{%` (or `use_jinja=True`), else `{var}` substitution (`use_jinja=False`
    forces it); a missing variable is an error."""
    if use_jinja or (use_jinja is None and ("{{" in template or "{%" in template)):
        try:
            import jinja2
            return jinja2.Environment(undefined=jinja2.StrictUndefined).from_string(template).render(**variables)
        except Exception as e:   # noqa: BLE001
            raise TemplateRenderError("jinja template failed", cause=e)

    def sub(m):
        k = m.group(1)
        if k not in variables:
            raise TemplateRenderError(f"template variable {k!r} is missing", available=sorted(variables))
        return str(variables[k])

    return _VAR.sub(sub, template)


class _LabelBuilder:
    @staticmethod
    def full_causal(ids: Sequence[int], mask: Sequence[int]) -> list[int]:
        return [t if m else IGNORE for t, m in zip(ids, mask)]

    @staticmethod
    def mask_prefix(ids: Sequence[int], mask: Sequence[int], prefix_len: int) -> list[int]:
        return [IGNORE if (i < prefix_len or not m) else t for i, (t, m) in enumerate(zip(ids, mask))]

    @staticmethod
    def mask_ranges(ids: Sequence[int], mask: Sequence[int], train_ranges: Iterable[tuple[int, int]]) -> list[int]:
        out = [IGNORE] * len(ids)
        for a, b in train_ranges:
            for i in range(max(0, a), min(len(ids), b)):
                if mask[i]:
                    out[i] = ids[i]
        return out

    @staticmethod
    def from_turn_boundaries(ids, mask, boundaries: Sequence[tuple[int, int, str]], train_roles: Sequence[str]):
        return _LabelBuilder.mask_ranges(ids, mask, [(a, b) for a, b, role in boundaries if role in train_roles])


class _Encoder:
    """Tokenisation helpers shared by the stage processors (ids without padding; pad / truncate at the end)."""

    def __init__(self, tok: TokenizerWrapper, max_length: int, pad_to_max: bool = True):
        self.tok, self.max_length, self.pad_to_max = tok, max_length, pad_to_max

    def ids(self, text: str) -> list[int]:
        return self.tok.encode_raw(text, add_special_tokens=False)

    def finish(self, ids: list[int], labels: list[int] | None = None, max_length: int | None = None,
               pad: bool | None = None) -> tuple[list[int], list[int], list[int]]:
        n = max_length or self.max_length
        ids = list(ids[:n])
        labels = list(labels[:n]) if labels is not None else list(ids)
        mask = [1] * len(ids)
        if (self.pad_to_max if pad is None else pad) and len(ids) < n:
            k = n - len(ids)
            ids += [self.tok.pad_token_id] * k
            labels += [IGNORE] * k
            mask += [0] * k
        return ids, mask, labels

    def apply_chat_template(self, messages: list[dict], add_generation_prompt=False) -> str:
        return self.tok.apply_chat_template(messages, add_generation_prompt)

    # ---- small accessors (data_pipeline/preprocessing/prompt_engine.py:_Encoder)
    pad_token_id = property(lambda self: self.tok.pad_token_id)
    eos_token_id = property(lambda self: self.tok.eos_token_id)
    eos_token = property(lambda self: getattr(self.tok.tokenizer, "eos_token", None) or "")
    bos_token = property(lambda self: getattr(self.tok.tokenizer, "bos_token", None) or "")

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return self.tok.encode_raw(text, add_special_tokens=add_special_tokens)

    def token_count(self, text: str) -> int:
        return len(self.ids(text))

    def encode_padded(self, text: str, max_length: int | None = None) -> tuple[list[int], list[int]]:
        """(input_ids, attention_mask), truncated and padded to `max_length`."""
        ids, mask, _ = self.finish(self.ids(text), None, max_length, pad=True)
        return ids, mask


# ------------------------------------------------------------------------------------------------ packing
def _greedy_pack(lengths: Sequence[int], capacity: int, max_per_pack: int = 0) -> list[list[int]]:
    bins, cur, used = [], [], 0
    for i, n in enumerate(lengths):
        if cur and (used + n > capacity or (max_per_pack and len(cur) >= max_per_pack)):
            bins.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += n
    if cur:
        bins.append(cur)
    return bins


def _ffd_pack(lengths: Sequence[int], capacity: int, max_per_pack: int = 0) -> list[list[int]]:
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: list[list[int]] = []
    free: list[int] = []
    for i in order:
        n = lengths[i]
        for b in range(len(bins)):
            if free[b] >= n and (not max_per_pack or len(bins[b]) < max_per_pack):
                bins[b].append(i)
                free[b] -= n
                break
        else:
            bins.append([i])
            free.append(capacity - n)
    return bins


def pack_token_documents(docs: Sequence[Sequence[int]], max_length: int, pad_token_id: int, cfg: PackingConfig | None = None,
                         eos_token_id: int | None = None, labels: Sequence[Sequence[int]] | None = None
                         ) -> list[PackedExample]:
    """Pack tokenised documents into sequences of `max_length` tokens (documents longer than that are split)."""
    cfg = cfg or PackingConfig(enabled=True)
    cap = cfg.max_packed_length or max_length
    sep = list(cfg.separator_tokens) or ([eos_token_id] if (cfg.add_eos_separator and eos_token_id is not None) else [])
    pieces, piece_labels = [], []
    for di, d in enumerate(docs):
        d = list(d)
        lab = list(labels[di]) if labels is not None else list(d)
        if sep and (not d or d[-len(sep):] != sep):
            d, lab = d + sep, lab + sep
        for s in range(0, len(d), cap):
            pieces.append(d[s:s + cap])
            piece_labels.append(lab[s:s + cap])
    lengths = [len(p) for p in pieces]
    strategy = PackingStrategy(cfg.strategy)
    if strategy == PackingStrategy.SINGLE:
        bins = [[i] for i in range(len(pieces))]
    elif strategy == PackingStrategy.FFD:
        bins = _ffd_pack(lengths, cap, cfg.max_sequences_per_pack)
    else:
        bins = _greedy_pack(lengths, cap, cfg.max_sequences_per_pack)
    out = []
    for b in bins:
        ids, lab, pos, doc, cu = [], [], [], [], [0]
        for k, i in enumerate(b):
            ids += pieces[i]
            lab += piece_labels[i]
            pos += list(range(lengths[i]))
            doc += [k] * lengths[i]
            cu.append(len(ids))
        fill = len(ids) / cap
        if cfg.drop_remainder and fill < 1.0 and b is bins[-1] and len(bins) > 1:
            continue
        if cfg.min_fill_ratio and fill < cfg.min_fill_ratio:
            continue
        mask = [1] * len(ids)
        k = cap - len(ids)
        if k > 0:
            ids += [pad_token_id] * k
            lab += [IGNORE] * k
            pos += [0] * k
            doc += [-1] * k
            mask += [0] * k
        out.append(PackedExample(ids, mask, lab, pos if cfg.add_position_ids else [], doc, len(b),
                                 cu if cfg.use_vsl else []))
    return out


# ------------------------------------------------------------------------------------------------ stage processors
class _PreTrainingProcessor:
    def __init__(self, cfg: PromptEngineConfig, enc: _Encoder):
        self.cfg, self.pt, self.enc = cfg, cfg.pre_training, enc
        self.rng = random.Random(self.pt.fim.seed)
        fim = self.pt.fim
        if fim.enabled or self.pt.format == PreTrainingFormat.FILL_IN_MIDDLE:
            enc.tok.add_special_tokens_dict({"additional_special_tokens": [fim.prefix_token, fim.suffix_token,
                                                                           fim.middle_token]})

    def process(self, row: Mapping[str, Any]) -> ProcessedExample:
        text = row.get(self.pt.text_column)
        if not isinstance(text, str):
            raise TokenizationError(f"column {self.pt.text_column!r} is missing or not text", columns=sorted(row))
        fmt = self.pt.format
        if fmt == PreTrainingFormat.SPAN_CORRUPTION or self.pt.span_corruption.enabled:
            return self._span_corruption(text)
        if fmt == PreTrainingFormat.FILL_IN_MIDDLE or self.pt.fim.enabled:
            return self._fill_in_middle(text)
        return self._causal_lm(text)

    def tokens(self, text: str) -> list[int]:
        tok = self.enc.tok
        ids = self.enc.ids(text)
        if self.pt.add_bos and tok.bos_token_id is not None:
            ids = [tok.bos_token_id] + ids
        if self.pt.add_eos and tok.eos_token_id is not None:
            ids = ids + [tok.eos_token_id]
        return ids

    def _causal_lm(self, text: str) -> ProcessedExample:
        ids, mask, labels = self.enc.finish(self.tokens(text))
        return ProcessedExample(ids, mask, labels)

    def _fill_in_middle(self, text: str) -> ProcessedExample:
        fim = self.pt.fim
        if self.rng.random() >= fim.fim_rate or len(text) < 3:
            return self._causal_lm(text)
        max_mid = max(1, int(len(text) * fim.max_middle_ratio))
        mid_len = self.rng.randint(1, max_mid)
        start = self.rng.randint(0, len(text) - mid_len)
        pre, mid, suf = text[:start], text[start:start + mid_len], text[start + mid_len:]
        spm = fim.mode == FIMMode.SPM or self.rng.random() < fim.spm_rate
        if spm:
            s = f"{fim.prefix_token}{fim.suffix_token}{suf}{fim.middle_token}{pre}{mid}"
        else:
            s = f"{fim.prefix_token}{pre}{fim.suffix_token}{suf}{fim.middle_token}{mid}"
        ex = self._causal_lm(s)
        ex.extras["fim"] = 1
        return ex

    def _span_corruption(self, text: str) -> ProcessedExample:
        sc = self.pt.span_corruption
        tok = self.enc.tok
        ids = self.enc.ids(text)
        rng = random.Random(sc.seed + len(ids))
        n = len(ids)
        first_sentinel = sc.sentinel_start if sc.sentinel_start is not None else tok.vocab_size - 1
        n_noise = max(1, int(round(n * sc.noise_density)))
        n_spans = max(1, min(sc.num_sentinels, int(round(n_noise / sc.mean_span_len))))
        starts = sorted(rng.sample(range(max(1, n - int(sc.mean_span_len))), min(n_spans, max(1, n - int(sc.mean_span_len)))))
        corrupted, targets, cursor, s_id = [], [], 0, 0
        for st in starts:
            if st < cursor:
                continue
            ln = max(1, int(rng.expovariate(1.0 / sc.mean_span_len)) or 1)
            ln = min(ln, n - st)
            sent = first_sentinel - s_id
            corrupted += ids[cursor:st] + [sent]
            targets += [sent] + ids[st:st + ln]
            cursor = st + ln
            s_id += 1
        corrupted += ids[cursor:]
        eos = [tok.eos_token_id] if tok.eos_token_id is not None else []
        full = corrupted + eos + targets + eos
        labels = [IGNORE] * (len(corrupted) + len(eos)) + targets + eos
        ids2, mask, labels = self.enc.finish(full, labels)
        return ProcessedExample(ids2, mask, labels, {"num_spans": s_id})

    def pack_documents(self, texts: Sequence[str], cfg: PackingConfig | None = None) -> list[PackedExample]:
        cfg = cfg or self.pt.packing
        docs = [self.tokens(t) for t in texts]
        # the separator is already the EOS appended by tokens(); avoid doubling it
        import dataclasses
        cfg = dataclasses.replace(cfg, add_eos_separator=cfg.add_eos_separator and not self.pt.add_eos)
        return pack_token_documents(docs, self.cfg.max_length, self.enc.tok.pad_token_id, cfg, self.enc.tok.eos_token_id)


class _FineTuningProcessor:
    def __init__(self, cfg: PromptEngineConfig, enc: _Encoder, template: PromptTemplate | None):
        self.cfg, self.ft, self.enc, self.template = cfg, cfg.fine_tuning, enc, template or PromptTemplate()

    def process(self, row: Mapping[str, Any]) -> ProcessedExample:
        fmt = FineTuningFormat(self.ft.format)
        return {FineTuningFormat.CHAT: self._chat, FineTuningFormat.COMPLETION: self._completion,
                FineTuningFormat.INSTRUCTION: self._instruction, FineTuningFormat.MULTI_TURN: self._multi_turn,
                FineTuningFormat.CUSTOM: self._custom}[fmt](row)

    def _pair(self, prompt: str, answer: str, mask_prompt: bool | None = None) -> ProcessedExample:
        tok = self.enc.tok
        p_ids = self.enc.ids(prompt)
        if self.template.add_bos and tok.bos_token_id is not None:
            p_ids = [tok.bos_token_id] + p_ids
        a_ids = self.enc.ids(answer)
        if self.template.add_eos and tok.eos_token_id is not None:
            a_ids = a_ids + [tok.eos_token_id]
        n = self.cfg.max_length
        if len(p_ids) + len(a_ids) > n:   # keep the answer, trim the prompt from the left, then the answer
            keep_p = max(0, n - len(a_ids))
            p_ids = p_ids[len(p_ids) - keep_p:] if keep_p else []
            a_ids = a_ids[:n - len(p_ids)]
        ids = p_ids + a_ids
        mp = self.ft.mask_prompt if mask_prompt is None else mask_prompt
        labels = ([IGNORE] * len(p_ids) if mp else list(p_ids)) + list(a_ids)
        ids, mask, labels = self.enc.finish(ids, labels)
        return ProcessedExample(ids, mask, labels, {"prompt_length": len(p_ids)})

    def _chat(self, row) -> ProcessedExample:
        t = self.template
        msgs = []
        if t.system_message:
            msgs.append({"role": "system", "content": t.system_message})
        user_cols = t.input_columns or (self.ft.prompt_column,)
        vars_ = {c: row.get(c, "") for c in row}
        user = render_template(t.user_template, vars_) if t.user_template else "\n".join(str(row.get(c, "")) for c in user_cols)
        answer_col = t.label_column or self.ft.completion_column
        answer = render_template(t.assistant_template, vars_) if t.assistant_template else str(row.get(answer_col, ""))
        msgs.append({"role": "user", "content": user})
        prompt = self.enc.apply_chat_template(msgs, add_generation_prompt=True)
        return self._pair(prompt, answer, t.mask_input)

    def _completion(self, row) -> ProcessedExample:
        return self._pair(str(row.get(self.ft.prompt_column, "")), str(row.get(self.ft.completion_column, "")))

    def _instruction(self, row) -> ProcessedExample:
        ins, inp = str(row.get(self.ft.instruction_column, "")), str(row.get(self.ft.input_column, "") or "")
        if inp:
            prompt = ("Below is an instruction that describes a task, paired with an input that provides further "
                      f"context. Write a response that appropriately completes the request.\n\n### Instruction:\n{ins}"
                      f"\n\n### Input:\n{inp}\n\n### Response:\n")
        else:
            prompt = ("Below is an instruction that describes a task. Write a response that appropriately completes "
                      f"the request.\n\n### Instruction:\n{ins}\n\n### Response:\n")
        return self._pair(prompt, str(row.get(self.ft.output_column, "")))

    def _multi_turn(self, row) -> ProcessedExample:
        mt = self.ft.multi_turn
        msgs = list(row.get(mt.messages_column) or [])
        if mt.system_message and not (msgs and msgs[0].get(mt.role_key) == "system"):
            msgs = [{mt.role_key: "system", mt.content_key: mt.system_message}] + msgs
        tok = self.enc.tok
        ids, bounds = [], []
        if self.template.add_bos and tok.bos_token_id is not None:
            ids.append(tok.bos_token_id)
        for m in msgs:
            role, content = m.get(mt.role_key, "user"), str(m.get(mt.content_key, ""))
            head = self.enc.ids(f"<|{role}|>\n")
            body = self.enc.ids(content + "\n")
            if role in mt.train_on_roles and tok.eos_token_id is not None:
                body = body + [tok.eos_token_id]
            ids += head
            bounds.append((len(ids), len(ids) + len(body), role))
            ids += body
        ids = ids[:self.cfg.max_length]
        labels = _LabelBuilder.from_turn_boundaries(ids, [1] * len(ids), bounds, mt.train_on_roles)
        ids, mask, labels = self.enc.finish(ids, labels)
        return ProcessedExample(ids, mask, labels, {"num_turns": len(msgs)})

    def _custom(self, row) -> ProcessedExample:
        t = self.template
        if not t.template:
            cols = t.input_columns or tuple(c for c in row if isinstance(row[c], str) and c != t.label_column)
            prompt = "\n".join(str(row.get(c, "")) for c in cols)
        else:
            prompt = render_template(t.template, dict(row))
        if t.label_column:
            return self._pair(prompt, str(row.get(t.label_column, "")), t.mask_input)
        ids = self.enc.ids(prompt)
        tok = self.enc.tok
        if t.add_eos and tok.eos_token_id is not None:
            ids = ids + [tok.eos_token_id]
        ids, mask, labels = self.enc.finish(ids)
        return ProcessedExample(ids, mask, labels)


class _RLProcessor:
    def __init__(self, cfg: PromptEngineConfig, enc: _Encoder):
        self.cfg, self.rl, self.enc = cfg, cfg.rl, enc
        self.c = cfg.rl.columns

    def _prompt_ids(self, prompt) -> list[int]:
        if isinstance(prompt, list):   # chat-style prompt
            prompt = self.enc.apply_chat_template(prompt, add_generation_prompt=True)
        ids = self.enc.ids(str(prompt))
        if self.rl.max_prompt_length:
            ids = ids[-self.rl.max_prompt_length:]
        return ids

    def _response_ids(self, resp) -> list[int]:
        if isinstance(resp, list):
            resp = resp[-1].get("content", "") if resp else ""
        ids = self.enc.ids(str(resp))
        eos = self.enc.tok.eos_token_id
        if eos is not None:
            ids = ids + [eos]
        if self.rl.max_response_length:
            ids = ids[:self.rl.max_response_length]
        return ids

    def _build_prompt_response_sequence(self, p_ids: list[int], r_ids: list[int]):
        n = self.cfg.max_length
        ids = (p_ids + r_ids)[:n]
        labels = ([IGNORE] * len(p_ids) + r_ids)[:n]
        return self.enc.finish(ids, labels, pad=True)

    def process(self, row: Mapping[str, Any]):
        return {RLAlgorithm.DPO: self._dpo, RLAlgorithm.ORPO: self._dpo, RLAlgorithm.REWARD_MODEL: self._dpo,
                RLAlgorithm.PPO: self._ppo, RLAlgorithm.KTO: self._kto, RLAlgorithm.GRPO: self._grpo}[
            RLAlgorithm(self.rl.algorithm)](row)

    def _dpo(self, row) -> PreferencePairExample:
        p = self._prompt_ids(row.get(self.c.prompt, ""))
        ci, cm, cl = self._build_prompt_response_sequence(p, self._response_ids(row.get(self.c.chosen, "")))
        ri, rm, rl_ = self._build_prompt_response_sequence(p, self._response_ids(row.get(self.c.rejected, "")))
        pi, pm, _ = self.enc.finish(p, pad=True, max_length=self.rl.max_prompt_length or self.cfg.max_length)
        return PreferencePairExample(pi, pm, ci, cm, cl, ri, rm, rl_)

    def _ppo(self, row) -> PPOExample:
        p = self._prompt_ids(row.get(self.c.prompt, ""))
        n = self.rl.max_prompt_length or self.cfg.max_length
        p = p[-n:]
        pad = [self.enc.tok.pad_token_id] * (n - len(p))   # left padding: generation continues on the right
        return PPOExample(pad + p, [0] * len(pad) + [1] * len(p), str(row.get(self.c.prompt, "")))

    def _kto(self, row) -> KTOExample:
        p = self._prompt_ids(row.get(self.c.prompt, ""))
        ids, mask, labels = self._build_prompt_response_sequence(p, self._response_ids(row.get(self.c.response,
                                                                                               row.get(self.c.chosen, ""))))
        tag = bool(row.get(self.c.label, True))
        return KTOExample(ids, mask, labels, tag, self.rl.desirable_weight if tag else self.rl.undesirable_weight)

    def _grpo(self, row) -> GRPOExample:
        p = self._prompt_ids(row.get(self.c.prompt, ""))
        responses = list(row.get(self.c.responses) or [])
        scores = [float(s) for s in (row.get(self.c.scores) or [0.0] * len(responses))]
        ri, rm, rl_ = [], [], []
        for r in responses:
            a, b, c = self._build_prompt_response_sequence(p, self._response_ids(r))
            ri.append(a)
            rm.append(b)
            rl_.append(c)
        pi, pm, _ = self.enc.finish(p, pad=True, max_length=self.rl.max_prompt_length or self.cfg.max_length)
        return GRPOExample(pi, pm, ri, rm, rl_, scores)


# ------------------------------------------------------------------------------------------------ facade
class PromptEngine:
    def __init__(self, config: PromptEngineConfig, tokenizer, distributor=None, template: PromptTemplate | None = None):
        self.config = config
        self.tokenizer = tokenizer if isinstance(tokenizer, TokenizerWrapper) else TokenizerWrapper(tokenizer)
        self.distributor = distributor
        self.template = template
        self.enc = _Encoder(self.tokenizer, config.max_length, config.pad_to_max_length)
        stage = TrainingStage(config.stage)
        if stage == TrainingStage.PRE_TRAINING:
            self.processor = _PreTrainingProcessor(config, self.enc)
        elif stage == TrainingStage.FINE_TUNING:
            self.processor = _FineTuningProcessor(config, self.enc, template)
        else:
            self.processor = _RLProcessor(config, self.enc)

    @property
    def stage(self) -> TrainingStage:
        return TrainingStage(self.config.stage)

    @property
    def max_length(self) -> int:
        return self.config.max_length

    @classmethod
    def from_config(cls, config: PromptEngineConfig, tokenizer, distributor=None, template=None) -> "PromptEngine":
        return cls(config, tokenizer, distributor, template)

    @classmethod
    def from_legacy(cls, template: PromptTemplate, tokenizer, max_length: int = 2048, distributor=None, *,
                    length_manager=None, per_column_limits: Mapping[str, int] | None = None) -> "PromptEngine":
        """Build from a bare `prompt_template` section (no `prompt_engine` block in the YAML).  `length_manager` (a
        LengthManager) or `per_column_limits` ({column: max tokens}) trim the row's text columns before templating, when
        no distributor does."""
        if distributor is None and (length_manager is not None or per_column_limits):
            from .length_manager import create_length_manager
            lm = length_manager if length_manager is not None else create_length_manager(
                max_total_length=max_length, per_column_limits=dict(per_column_limits), tokenizer=tokenizer)

            class _Trim:
                def distribute(self, row):
                    return lm.preprocess_example({k: v for k, v in row.items() if isinstance(v, str)}) | \
                        {k: v for k, v in row.items() if not isinstance(v, str)}
            distributor = _Trim()
        import dataclasses
        fmt = {"chat": FineTuningFormat.CHAT, "completion": FineTuningFormat.COMPLETION}.get(template.format_type,
                                                                                              FineTuningFormat.CUSTOM)
        cfg = PromptEngineConfig(stage=TrainingStage.FINE_TUNING, max_length=max_length)
        cfg = dataclasses.replace(cfg, fine_tuning=dataclasses.replace(cfg.fine_tuning, format=fmt,
                                                                       mask_prompt=template.mask_input))
        return cls(cfg, tokenizer, distributor, template)

    def _preprocess_example(self, row: Mapping[str, Any]) -> dict:
        row = dict(row)
        for src, dst in (self.config.column_mapping or {}).items():
            if src in row and dst not in row:
                row[dst] = row[src]
        for col, lim in (self.config.per_column_limits or {}).items():
            if isinstance(row.get(col), str):
                from .length_manager import smart_truncate
                row[col] = smart_truncate(row[col], int(lim * 3.8), self.config.truncation_strategy)
        if self.distributor is not None:
            row = self.distributor.distribute(row)
        return row

    @reference_kwargs(example="row")
    def process(self, row: Mapping[str, Any]):
        return self.processor.process(self._preprocess_example(row))

    @reference_kwargs(examples="rows")
    def process_batch(self, rows: Iterable[Mapping[str, Any]], skip_errors: bool = False) -> list:
        out = []
        for r in rows:
            try:
                out.append(self.process(r))
            except (TokenizationError, TemplateRenderError):
                if not skip_errors:
                    raise
        return out

    @reference_kwargs(examples="texts")
    def pack_documents(self, texts: Sequence, packing: PackingConfig | None = None) -> list[PackedExample]:
        """`texts`: strings, or rows (mappings) from which the configured text column is taken."""
        if not isinstance(self.processor, _PreTrainingProcessor):
            raise TokenizationError("pack_documents needs a pre_training prompt engine")
        if texts and isinstance(texts[0], Mapping):
            col = getattr(getattr(self.config, "pre_training", None), "text_column", "text")
            texts = [t[col] for t in texts]
        return self.processor.pack_documents(texts, packing)

    def describe(self) -> dict:
        return {"stage": TrainingStage(self.config.stage).value, "max_length": self.config.max_length,
                "processor": type(self.processor).__name__, "vocab_size": self.tokenizer.vocab_size}


def batch_to_dict(examples: Sequence) -> dict[str, torch.Tensor]:
    """List of example containers -> dict of stacked LongTensors (ragged / scalar fields become tensors or lists)."""
    dicts = [e.to_dict() if hasattr(e, "to_dict") else dict(e) for e in examples]
    out = {}
    for k in dicts[0]:
        vals = [d[k] for d in dicts]
        try:
            out[k] = torch.tensor(vals)
        except (ValueError, TypeError, RuntimeError):
            out[k] = vals
    return out


def create_dataset_map_fn(engine: PromptEngine, drop_errors: bool = False) -> Callable[[Mapping[str, Any]], dict]:
    """Function for `datasets.Dataset.map`: row -> plain dict of lists.  With `drop_errors` a row that cannot be
    processed maps to empty lists (filter on `len(input_ids) > 0` afterwards) instead of raising."""
    def fn(row):
        try:
            return engine.process(row).to_dict()
        except PipelineError:
            if not drop_errors:
                raise
            return {"input_ids": [], "attention_mask": [], "labels": []}
    return fn


# convenience factories mirroring the reference's module-level helpers
def create_pretraining_engine(tokenizer, max_length=2048, fmt="causal_lm", text_column="text", **pt_kw) -> PromptEngine:
    import dataclasses
    from ..config.data_schema import PreTrainingConfig
    pt = PreTrainingConfig(format=PreTrainingFormat(fmt), text_column=text_column, **pt_kw)
    return PromptEngine(PromptEngineConfig(stage=TrainingStage.PRE_TRAINING, max_length=max_length, pre_training=pt), tokenizer)


def create_finetuning_engine(tokenizer, max_length=2048, fmt="instruction", template: PromptTemplate | None = None,
                             **ft_kw) -> PromptEngine:
    from ..config.data_schema import FineTuningConfig
    ft = FineTuningConfig(format=FineTuningFormat(fmt), **ft_kw)
    return PromptEngine(PromptEngineConfig(stage=TrainingStage.FINE_TUNING, max_length=max_length, fine_tuning=ft),
                        tokenizer, template=template)


def create_rl_engine(tokenizer, max_length=2048, algorithm="dpo", **rl_kw) -> PromptEngine:
    from ..config.data_schema import RLConfig
    rl = RLConfig(algorithm=RLAlgorithm(algorithm), **rl_kw)
    return PromptEngine(PromptEngineConfig(stage=TrainingStage.POST_TRAINING, max_length=max_length, rl=rl), tokenizer)


def extract_successful(results):
    """Split a list of Results into (ok values, errors), keeping order."""
    oks, errs = [], []
    for r in results:
        if r.is_ok():
            oks.append(r.unwrap())
        else:
            errs.append(r.error)
    return oks, errs


# ---- names of data_pipeline/preprocessing/prompt_engine.py
import re as _re  # noqa: E402
from typing import Union as _Union  # noqa: E402

LABEL_PAD_TOKEN_ID: int = -100
SIMPLE_VAR_PATTERN = _re.compile(r"\{(\w+)\}")             # {name} placeholders of the non-Jinja templates
ProcessedOutput = _Union[ProcessedExample, PackedExample, PreferencePairExample, PPOExample, KTOExample, GRPOExample]
