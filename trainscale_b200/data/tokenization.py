"""Tokenizer wrapper: a uniform encode / decode / count surface over HuggingFace tokenizers, plus a built-in
byte-level tokenizer so that pipelines, tests and synthetic runs work with no files and no network.

Surface after data_pipeline/preprocessing/tokenization.py:88-913 (`_resolve_token_id`, pad-token repair,
`TokenizerWrapper.encode / encode_batch / encode_raw / count_tokens / decode / get_special_tokens_mask`,
vocabulary-growth tracking, `create_tokenizer`, `wrap_tokenizer`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Iterable, Sequence

import torch

from ..utils.refargs import ANY, reference_kwargs

from ..core.errors import TokenizationError


class ByteTokenizer:
    """UTF-8 byte tokenizer: ids 0..255 are bytes, then <pad>=256 <bos>=257 <eos>=258 <unk>=259, then added tokens."""

    def __init__(self, extra_tokens: Sequence[str] = ()):
        self.special = {"<pad>": 256, "<bos>": 257, "<eos>": 258, "<unk>": 259}
        self.added: dict[str, int] = {}
        self.pad_token, self.bos_token, self.eos_token, self.unk_token = "<pad>", "<bos>", "<eos>", "<unk>"
        self.padding_side, self.truncation_side = "right", "right"
        self.chat_template = None
        self.name_or_path = "byte"
        self.add_tokens(list(extra_tokens))

    # --- ids
    @property
    def pad_token_id(self): return self.special["<pad>"]
    @property
    def bos_token_id(self): return self.special["<bos>"]
    @property
    def eos_token_id(self): return self.special["<eos>"]
    @property
    def unk_token_id(self): return self.special["<unk>"]
    @property
    def vocab_size(self): return 260
    def __len__(self): return 260 + len(self.added)

    def add_tokens(self, toks: Sequence[str]) -> int:
        n = 0
        for t in toks:
            if t not in self.added and t not in self.special:
                self.added[t] = 260 + len(self.added)
                n += 1
        return n

    def add_special_tokens(self, d: dict) -> int:
        toks = []
        for v in d.values():
            toks += list(v) if isinstance(v, (list, tuple)) else [v]
        return self.add_tokens([t for t in toks if isinstance(t, str)])

    def convert_tokens_to_ids(self, tok):
        if isinstance(tok, (list, tuple)):
            return [self.convert_tokens_to_ids(t) for t in tok]
        if tok in self.special or tok in self.added:
            return self.special.get(tok, self.added.get(tok))
        # byte tokens are spelled as the character of that code (the inverse of convert_ids_to_tokens)
        return ord(tok) if isinstance(tok, str) and len(tok) == 1 and ord(tok) < 256 else self.unk_token_id

    def convert_ids_to_tokens(self, i):
        if isinstance(i, (list, tuple)):
            return [self.convert_ids_to_tokens(x) for x in i]
        inv = {v: k for k, v in {**self.special, **self.added}.items()}
        return inv.get(i, chr(i) if i < 256 else "<unk>")

    def _encode_text(self, text: str) -> list[int]:
        table = {**self.special, **self.added}
        if not table:
            return list(text.encode("utf-8"))
        out, i = [], 0
        keys = sorted(table, key=len, reverse=True)
        while i < len(text):
            if text[i] == "<":
                hit = next((k for k in keys if text.startswith(k, i)), None)
                if hit is not None:
                    out.append(table[hit])
                    i += len(hit)
                    continue
            out.extend(text[i].encode("utf-8"))
            i += 1
        return out

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        ids = self._encode_text(text)
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = True) -> str:
        inv = {v: k for k, v in {**self.special, **self.added}.items()}
        buf, out = bytearray(), []
        for i in ids:
            i = int(i)
            if i < 256:
                buf.append(i)
            else:
                if buf:
                    out.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                if not skip_special_tokens:
                    out.append(inv.get(i, ""))
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def __call__(self, text, add_special_tokens=True, truncation=False, max_length=None, padding=False,
                 return_attention_mask=True, **_):
        texts = [text] if isinstance(text, str) else list(text)
        rows = []
        for t in texts:
            ids = self.encode(t, add_special_tokens)
            if truncation and max_length is not None and len(ids) > max_length:
                ids = ids[-max_length:] if self.truncation_side == "left" else ids[:max_length]
            rows.append(ids)
        width = max_length if padding == "max_length" and max_length else (max(map(len, rows)) if padding else None)
        masks = []
        for k, ids in enumerate(rows):
            m = [1] * len(ids)
            if width is not None and len(ids) < width:
                pad = [self.pad_token_id] * (width - len(ids))
                ids, m = (pad + ids, [0] * len(pad) + m) if self.padding_side == "left" else (ids + pad, m + [0] * len(pad))
            rows[k] = ids
            masks.append(m)
        out = {"input_ids": rows if not isinstance(text, str) else rows[0]}
        if return_attention_mask:
            out["attention_mask"] = masks if not isinstance(text, str) else masks[0]
        return out


def _resolve_token_id(tok, token) -> int | None:
    """A token given as id, string or None -> id (None when the tokenizer does not know it)."""
    if token is None:
        return None
    if isinstance(token, int):
        return token
    i = tok.convert_tokens_to_ids(token)
    unk = getattr(tok, "unk_token_id", None)
    if i is None or (unk is not None and i == unk and token != getattr(tok, "unk_token", None)):
        return None
    return i


def _ensure_pad_token(tok) -> str:
    """Make sure a pad token exists: reuse eos, then unk, else add '<pad>'. Returns how it was resolved."""
    if getattr(tok, "pad_token", None) is not None and getattr(tok, "pad_token_id", None) is not None:
        return "existing"
    if getattr(tok, "eos_token", None) is not None:
        tok.pad_token = tok.eos_token
        return "eos"
    if getattr(tok, "unk_token", None) is not None:
        tok.pad_token = tok.unk_token
        return "unk"
    tok.add_special_tokens({"pad_token": "<pad>"})
    return "added"


@dataclass
class Encoding:
    input_ids: list[int]
    attention_mask: list[int]

    def __len__(self):
        return len(self.input_ids)


class TokenizerWrapper:
    def __init__(self, tokenizer, max_length: int = 2048, padding: str | bool = "max_length", truncation: bool = True,
                 padding_side: str = "right", truncation_side: str = "right", add_special_tokens: bool = True,
                 special_tokens: dict | None = None, *, config=None, original_vocab_size: int | None = None,
                 vocab_was_modified: bool | None = None):
        """`config` (a TokenizerConfig) supplies the settings above; `original_vocab_size` is the vocabulary size before
        the caller added tokens itself (the reference passes it, with `vocab_was_modified`, when it loaded and extended
        the tokenizer before wrapping it); both are otherwise derived."""
        if config is not None and not isinstance(config, (int, float)):
            max_length = getattr(config, "max_length", max_length)
            padding, truncation = getattr(config, "padding", padding), getattr(config, "truncation", truncation)
            padding_side = getattr(config, "padding_side", padding_side)
            truncation_side = getattr(config, "truncation_side", truncation_side)
            add_special_tokens = getattr(config, "add_special_tokens", add_special_tokens)
            special_tokens = special_tokens or dict(getattr(config, "special_tokens", {}) or {})
        self.tokenizer = tokenizer
        self.max_length, self.padding, self.truncation = max_length, padding, truncation
        self.add_special_tokens = add_special_tokens
        tokenizer.padding_side, tokenizer.truncation_side = padding_side, truncation_side
        self.pad_resolution = _ensure_pad_token(tokenizer)
        self._initial_vocab = len(tokenizer) if original_vocab_size is None else int(original_vocab_size)
        if special_tokens:
            self.add_special_tokens_dict(special_tokens)

    # --- vocabulary growth (the model's embedding must be resized when this is > 0)
    def add_special_tokens_dict(self, d: dict) -> int:
        extra = {k: v for k, v in d.items() if v}
        if not extra:
            return 0
        if "additional_special_tokens" not in extra and any(k not in ("pad_token", "bos_token", "eos_token", "unk_token",
                                                                       "sep_token", "cls_token", "mask_token") for k in extra):
            extra = {"additional_special_tokens": [v for v in extra.values() if isinstance(v, str)]}
        return self.tokenizer.add_special_tokens(extra)

    @property
    def vocab_growth(self) -> int:
        return len(self.tokenizer) - self._initial_vocab

    @property
    def vocab_size(self) -> int:
        return len(self.tokenizer)

    @property
    def pad_token_id(self) -> int:
        return self.tokenizer.pad_token_id

    @property
    def eos_token_id(self):
        return getattr(self.tokenizer, "eos_token_id", None)

    @property
    def bos_token_id(self):
        return getattr(self.tokenizer, "bos_token_id", None)

    def token_id(self, token) -> int | None:
        return _resolve_token_id(self.tokenizer, token)

    # --- encoding
    def encode(self, text: str, max_length: int | None = None, padding=None, truncation=None,
               add_special_tokens: bool | None = None) -> Encoding:
        if not isinstance(text, str):
            raise TokenizationError("encode expects a string", got=type(text).__name__)
        try:
            out = self.tokenizer(text, add_special_tokens=self.add_special_tokens if add_special_tokens is None else add_special_tokens,
                                 truncation=self.truncation if truncation is None else truncation,
                                 max_length=max_length or self.max_length,
                                 padding=self.padding if padding is None else padding, return_attention_mask=True)
        except Exception as e:   # noqa: BLE001
            raise TokenizationError("tokenizer failed", cause=e, text_preview=text[:80])
        return Encoding(list(out["input_ids"]), list(out["attention_mask"]))

    def encode_batch(self, texts: Sequence[str], **kw) -> list[Encoding]:
        return [self.encode(t, **kw) for t in texts]

    def encode_raw(self, text: str, add_special_tokens: bool = False) -> list[int]:
        """ids only: no padding, no truncation."""
        out = self.tokenizer(text, add_special_tokens=add_special_tokens, truncation=False, padding=False,
                             return_attention_mask=False)
        return list(out["input_ids"])

    def count_tokens(self, text: str, add_special_tokens: bool = False) -> int:
        return len(self.encode_raw(text, add_special_tokens=add_special_tokens))

    @reference_kwargs({"clean_up_tokenization_spaces": ANY}, token_ids="ids")
    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        if torch.is_tensor(ids):
            ids = ids.tolist()
        return self.tokenizer.decode(ids, skip_special_tokens=skip_special_tokens)

    @reference_kwargs({"already_has_special_tokens": ANY}, token_ids="ids")
    def get_special_tokens_mask(self, ids: Sequence[int]) -> list[int]:
        special = {i for i in (self.pad_token_id, self.eos_token_id, self.bos_token_id,
                               getattr(self.tokenizer, "unk_token_id", None)) if i is not None}
        special |= set(getattr(self.tokenizer, "all_special_ids", []) or [])
        return [1 if int(i) in special else 0 for i in ids]

    # ---- vocabulary bookkeeping and conversions (data_pipeline/preprocessing/tokenization.py:332-356, 565-667)
    original_vocab_size = property(lambda self: self._initial_vocab)
    num_added_tokens = property(lambda self: max(0, len(self.tokenizer) - self._initial_vocab))
    vocab_was_modified = property(lambda self: len(self.tokenizer) != self._initial_vocab)

    def decode_batch(self, batch_token_ids, *, skip_special_tokens: bool = True) -> list[str]:
        return [self.decode(ids, skip_special_tokens) for ids in batch_token_ids]

    def get_all_special_token_ids(self) -> frozenset:
        """Every special token id the tokenizer knows (label masking: these positions usually get -100)."""
        ids = set(getattr(self.tokenizer, "all_special_ids", []) or [])
        for attr in ("pad", "eos", "bos", "unk", "sep", "cls", "mask"):
            i = getattr(self.tokenizer, f"{attr}_token_id", None)
            if i is not None:
                ids.add(int(i))
        return frozenset(ids)

    def get_special_tokens_info(self) -> dict:
        """{attribute: {"string": token, "id": id} or None} for the canonical special tokens."""
        info = {}
        for attr in ("pad_token", "eos_token", "bos_token", "unk_token", "sep_token", "cls_token", "mask_token"):
            tok = getattr(self.tokenizer, attr, None)
            info[attr] = None if tok is None else {"string": tok, "id": getattr(self.tokenizer, f"{attr}_id", None)}
        return info

    def convert_tokens_to_ids(self, tokens):
        fn = getattr(self.tokenizer, "convert_tokens_to_ids", None)
        if fn is not None:
            return fn(tokens)
        one = isinstance(tokens, str)
        out = [_resolve_token_id(self.tokenizer, t) for t in ([tokens] if one else tokens)]
        return out[0] if one else out

    def convert_ids_to_tokens(self, ids):
        fn = getattr(self.tokenizer, "convert_ids_to_tokens", None)
        if fn is not None:
            return fn(ids)
        one = isinstance(ids, int)
        out = [self.tokenizer.decode([i], skip_special_tokens=False) for i in ([ids] if one else ids)]
        return out[0] if one else out

    def __len__(self) -> int:
        return self.vocab_size

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = False) -> str:
        tok = self.tokenizer
        if getattr(tok, "chat_template", None) and hasattr(tok, "apply_chat_template"):
            return tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)
        text = "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in messages)
        return text + ("<|assistant|>\n" if add_generation_prompt else "")


def create_tokenizer(config=None, name_or_path: str | None = None, token: str | None = None,
                     trust_remote_code: bool = False, **overrides) -> TokenizerWrapper:
    """From a TokenizerConfig (or a name): 'byte' builds the built-in tokenizer, anything else goes through
    `transformers.AutoTokenizer` (local directory or hub)."""
    name = name_or_path or getattr(config, "name_or_path", None)
    if not name:
        raise TokenizationError("tokenizer name_or_path is required")
    kw = {}
    if config is not None:
        kw = dict(max_length=config.max_length, padding=config.padding, truncation=config.truncation,
                  padding_side=config.padding_side, truncation_side=config.truncation_side,
                  add_special_tokens=getattr(config, "add_special_tokens", True),
                  special_tokens=dict(getattr(config, "special_tokens", {}) or {}))
    kw.update(overrides)
    if str(name).lower() in ("byte", "bytes", "builtin:byte"):
        return TokenizerWrapper(ByteTokenizer(), **kw)
    try:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(name, token=token, trust_remote_code=trust_remote_code,
                                            use_fast=getattr(config, "use_fast", True))
    except Exception as e:   # noqa: BLE001
        raise TokenizationError(f"cannot load tokenizer {name!r}", cause=e)
    return TokenizerWrapper(tok, **kw)


def wrap_tokenizer(tokenizer, **kw) -> TokenizerWrapper:
    return tokenizer if isinstance(tokenizer, TokenizerWrapper) else TokenizerWrapper(tokenizer, **kw)


def ensure_tokenizer_padding(tokenizer) -> int:
    """Give a raw tokenizer a pad token if it has none (eos, then unk, else a new '<pad>') and return its id."""
    _ensure_pad_token(tokenizer)
    pid = getattr(tokenizer, "pad_token_id", None)
    if pid is None and hasattr(tokenizer, "convert_tokens_to_ids"):
        pid = tokenizer.convert_tokens_to_ids(tokenizer.pad_token)
    return int(pid if pid is not None else 0)
