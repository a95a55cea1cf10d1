"""Batch collation: pad by key suffix, re-mask labels on padding, causal-LM and seq2seq variants.

After data_pipeline/data/collate.py:50-393 (`pad_sequence_right/left`, picklable `CollateFn` with pad value chosen by
key suffix - `*input_ids` -> pad id, `*labels` -> -100, `*attention_mask` -> 0 - and labels <- -100 where the mask is 0).
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch
from ..utils.refargs import ANY, reference_kwargs

from ..core.errors import CollationError


@reference_kwargs(sequences="seqs", padding_value="pad_value")
def pad_sequence_right(seqs: Sequence[torch.Tensor], pad_value: int, max_length: int | None = None) -> torch.Tensor:
    n = max_length or max(len(s) for s in seqs)
    out = torch.full((len(seqs), n), pad_value, dtype=seqs[0].dtype)
    for i, s in enumerate(seqs):
        s = s[:n]
        out[i, :len(s)] = s
    return out


@reference_kwargs(sequences="seqs", padding_value="pad_value")
def pad_sequence_left(seqs: Sequence[torch.Tensor], pad_value: int, max_length: int | None = None) -> torch.Tensor:
    n = max_length or max(len(s) for s in seqs)
    out = torch.full((len(seqs), n), pad_value, dtype=seqs[0].dtype)
    for i, s in enumerate(seqs):
        s = s[-n:]
        out[i, n - len(s):] = s
    return out


class CollateFn:
    """Picklable (works with DataLoader worker processes)."""

    def __init__(self, pad_token_id: int = 0, label_pad_token_id: int = -100, padding_side: str = "right",
                 max_length: int | None = None, pad_values: Mapping[str, int] | None = None,
                 pad_to_multiple_of: int | None = None, output_schema=None, label_dtype: torch.dtype | None = None):
        """`output_schema` (a config OutputSchema) supplies per-key pad values; `label_dtype` casts every `*labels`
        tensor of the batch (e.g. torch.float for regression targets)."""
        self.pad_token_id, self.label_pad, self.side = pad_token_id, label_pad_token_id, padding_side
        self.max_length, self.pad_values, self.multiple = max_length, dict(pad_values or {}), pad_to_multiple_of
        self.label_dtype = label_dtype
        if output_schema is not None:
            for k, spec in getattr(output_schema, "tensors", {}).items():
                if k != "input_ids":
                    self.pad_values.setdefault(k, spec.pad_value)

    def _pad_value(self, key: str) -> int:
        if key in self.pad_values:
            return self.pad_values[key]
        if key.endswith("labels"):
            return self.label_pad
        if key.endswith("attention_mask"):
            return 0
        if key.endswith("document_ids"):
            return -1
        if key.endswith("input_ids"):
            return self.pad_token_id
        return 0

    def __call__(self, batch: Sequence[Mapping]) -> dict:
        if not batch:
            raise CollationError("empty batch")
        out = {}
        pad = pad_sequence_left if self.side == "left" else pad_sequence_right
        for key in batch[0]:
            vals = [b[key] for b in batch]
            if isinstance(vals[0], (str, bytes)) or vals[0] is None:
                out[key] = vals
                continue
            try:
                ts = [torch.as_tensor(v) for v in vals]
            except (ValueError, TypeError, RuntimeError):
                out[key] = vals
                continue
            if ts[0].dim() == 0:
                out[key] = torch.stack(ts)
            elif ts[0].dim() == 1:
                width = self.max_length or max(len(t) for t in ts)
                if self.multiple:
                    width = (width + self.multiple - 1) // self.multiple * self.multiple
                out[key] = pad(ts, self._pad_value(key), width)
            else:
                try:
                    out[key] = torch.stack(ts)
                except RuntimeError as e:
                    raise CollationError(f"cannot stack key {key!r}", cause=e)
        for key in list(out):   # labels never train on padding
            if key.endswith("labels") and torch.is_tensor(out[key]):
                mk = key[:-len("labels")] + "attention_mask"
                if mk in out and torch.is_tensor(out[mk]) and out[mk].shape == out[key].shape:
                    out[key] = out[key].masked_fill(out[mk] == 0, self.label_pad)
        if getattr(self, "label_dtype", None) is not None:
            for key in out:
                if key.endswith("labels") and torch.is_tensor(out[key]):
                    out[key] = out[key].to(self.label_dtype)
        if "document_ids" in out and torch.is_tensor(out["document_ids"]) and "cu_seqlens" not in out:
            from .packing import cu_seqlens_from_document_ids
            out["cu_seqlens"], out["max_seqlen"] = cu_seqlens_from_document_ids(out["document_ids"])
        return out


def create_collate_fn(pad_token_id: int = 0, label_pad_token_id: int = -100, padding_side: str = "right",
                      max_length: int | None = None, output_schema=None, **kw) -> CollateFn:
    pad_values = {}
    if output_schema is not None:
        pad_values = {k: spec.pad_value for k, spec in output_schema.tensors.items() if k not in ("input_ids",)}
    return CollateFn(pad_token_id, label_pad_token_id, padding_side, max_length, pad_values, **kw)


class _ShiftedCollate(CollateFn):
    def __call__(self, batch):
        out = super().__call__(batch)
        if "labels" not in out:
            out["labels"] = out["input_ids"].clone()
        lab = out["labels"]
        out["labels"] = torch.cat((lab[:, 1:], torch.full_like(lab[:, :1], self.label_pad)), dim=1)
        out["labels_shifted"] = True
        return out


def create_causal_lm_collate(pad_token_id: int = 0, shift_labels: "bool | int | None" = False, padding_side: str | None = None,
                             **kw) -> CollateFn:
    """Labels default to input_ids; with `shift_labels` they are pre-shifted (for models that do not shift).
    `create_causal_lm_collate(pad_token_id, max_length, padding_side)` is the positional form of
    data_pipeline/data/collate.py: an int (or None) in the second place is the maximum length."""
    if shift_labels is None or (isinstance(shift_labels, int) and not isinstance(shift_labels, bool)):
        if shift_labels is not None:
            kw.setdefault("max_length", shift_labels)
        shift_labels = False
    if padding_side is not None:
        kw.setdefault("padding_side", padding_side)
    return _ShiftedCollate(pad_token_id, **kw) if shift_labels else CollateFn(pad_token_id, **kw)


def create_seq2seq_collate(pad_token_id: int = 0, decoder_start_token_id: int = 0, **kw):
    base = CollateFn(pad_token_id, **kw)

    def fn(batch):
        out = base(batch)
        if "labels" in out and "decoder_input_ids" not in out:
            lab = out["labels"].masked_fill(out["labels"] == base.label_pad, pad_token_id)
            out["decoder_input_ids"] = torch.cat((torch.full_like(lab[:, :1], decoder_start_token_id), lab[:, :-1]), 1)
        return out

    return fn


# ---- defaults of the collators, by the names of data_pipeline/data/collate.py
DEFAULT_PAD_TOKEN_ID: int = 0
DEFAULT_LABEL_PAD_ID: int = -100           # the ignore_index of the cross-entropy kernels
DTYPE_MAP = {"long": torch.long, "int": torch.int, "float": torch.float, "half": torch.half,
             "bfloat16": torch.bfloat16, "bool": torch.bool}
