"""Trainer-side sequence packing over already tokenised examples.

After data_pipeline/trainer/packing.py:39-375: first-fit-decreasing over lengths, `pack_sequences` emitting
input_ids / attention_mask / labels / position_ids + `cu_seqlens` (int32), block-diagonal additive mask,
`unpack_sequences`, `PackedDataset`, `get_packing_stats`.  Here `cu_seqlens` feeds the variable-length flash
attention kernel directly (the reference emits it but has no kernel that consumes it).
"""
from __future__ import annotations

from typing import Sequence

import torch
from ..utils.refargs import ANY, reference_kwargs
from torch.utils.data import Dataset


@reference_kwargs(max_capacity="max_length")
def first_fit_decreasing(lengths: Sequence[int], max_length: int) -> list[list[int]]:
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins, free = [], []
    for i in order:
        n = min(lengths[i], max_length)
        for b in range(len(bins)):
            if free[b] >= n:
                bins[b].append(i)
                free[b] -= n
                break
        else:
            bins.append([i])
            free.append(max_length - n)
    return bins


@reference_kwargs(max_seq_len="max_length", label_pad_id="label_pad")
def pack_sequences(sequences: Sequence[dict] | None = None, max_length: int = 2048, pad_token_id: int = 0,
                   label_pad: int = -100, *more, input_ids=None, attention_mask=None, labels=None) -> list[dict]:
    """Each input dict holds 1-D `input_ids` (and optionally `labels`); returns packed dicts of tensors.  The
    reference's column form is taken too: `input_ids` / `attention_mask` / `labels` as lists (or padded [N, L] tensors)
    of the N sequences, the mask giving each row's real length."""
    if not isinstance(max_length, int) or more:
        # the reference's positional order: (input_ids, attention_mask, labels, max_seq_len, pad_token_id, label_pad_id)
        given = (max_length, pad_token_id, label_pad) + tuple(more)
        input_ids, attention_mask, labels = sequences, given[0], (given[1] if not isinstance(given[1], int) else None)
        tail = [g for g in given[2:] if isinstance(g, int)]
        max_length = tail[0] if tail else 2048
        pad_token_id = tail[1] if len(tail) > 1 else 0
        label_pad = tail[2] if len(tail) > 2 else -100
        sequences = None
    if sequences is None or input_ids is not None or (torch.is_tensor(sequences) and sequences.dim() == 2):
        ids = input_ids if input_ids is not None else sequences
        rows = []
        for i in range(len(ids)):
            n = int(torch.as_tensor(attention_mask[i]).sum()) if attention_mask is not None else len(ids[i])
            row = {"input_ids": torch.as_tensor(ids[i])[:n]}
            if labels is not None:
                row["labels"] = torch.as_tensor(labels[i])[:n]
            rows.append(row)
        sequences = rows
    lengths = [min(len(s["input_ids"]), max_length) for s in sequences]
    out = []
    for b in first_fit_decreasing(lengths, max_length):
        ids, labels, pos, cu = [], [], [], [0]
        for i in b:
            x = torch.as_tensor(sequences[i]["input_ids"])[:max_length]
            y = torch.as_tensor(sequences[i].get("labels", sequences[i]["input_ids"]))[:max_length]
            ids.append(x)
            labels.append(y)
            pos.append(torch.arange(len(x)))
            cu.append(cu[-1] + len(x))
        ids, labels, pos = torch.cat(ids), torch.cat(labels), torch.cat(pos)
        n = len(ids)
        pad = max_length - n
        mask = torch.cat((torch.ones(n, dtype=torch.long), torch.zeros(pad, dtype=torch.long)))
        if pad:
            ids = torch.cat((ids, torch.full((pad,), pad_token_id, dtype=ids.dtype)))
            labels = torch.cat((labels, torch.full((pad,), label_pad, dtype=labels.dtype)))
            pos = torch.cat((pos, torch.zeros(pad, dtype=pos.dtype)))
        doc = torch.full((max_length,), -1, dtype=torch.long)
        for k in range(len(b)):
            doc[cu[k]:cu[k + 1]] = k
        out.append({"input_ids": ids, "attention_mask": mask, "labels": labels, "position_ids": pos,
                    "document_ids": doc, "cu_seqlens": torch.tensor(cu, dtype=torch.int32), "source_indices": list(b)})
    return out


@reference_kwargs(max_seq_len="total_length")
def create_packed_attention_mask(cu_seqlens: torch.Tensor, total_length: int, dtype=torch.float32) -> torch.Tensor:
    """Block-diagonal causal additive mask [L, L]: 0 where attention is allowed, -inf elsewhere."""
    m = torch.full((total_length, total_length), float("-inf"), dtype=dtype)
    cu = cu_seqlens.tolist()
    for a, b in zip(cu[:-1], cu[1:]):
        n = b - a
        m[a:b, a:b] = torch.triu(torch.full((n, n), float("-inf"), dtype=dtype), diagonal=1)
    return m


@reference_kwargs(packed_output="packed")
def unpack_sequences(packed: torch.Tensor, cu_seqlens: torch.Tensor, original_lengths=None) -> list[torch.Tensor]:
    """Cut a packed row back into its sequences.  `original_lengths` (one per sequence) crops each piece to its
    length before packing (pieces are never longer than their segment)."""
    cu = cu_seqlens.tolist()
    out = [packed[..., a:b, :] if packed.dim() > 1 else packed[a:b] for a, b in zip(cu[:-1], cu[1:])]
    if original_lengths is not None:
        out = [(o[..., :int(n), :] if o.dim() > 1 else o[:int(n)]) for o, n in zip(out, original_lengths)]
    return out


class PackedDataset(Dataset):
    @reference_kwargs({"batch_size": ANY}, max_seq_len="max_length")      # batching is the DataLoader's job here
    def __init__(self, dataset, max_length: int, pad_token_id: int = 0, window: int = 1024):
        seqs = [dataset[i] for i in range(len(dataset))]
        self.items = []
        for s in range(0, len(seqs), window):   # pack inside windows so that memory stays bounded
            self.items += pack_sequences(seqs[s:s + window], max_length, pad_token_id)

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        d = dict(self.items[i])
        d.pop("source_indices", None)
        d.pop("cu_seqlens", None)   # ragged across items; rebuilt from document_ids by the collate function
        return d


def cu_seqlens_from_document_ids(document_ids: torch.Tensor) -> tuple[torch.Tensor, int]:
    """[B, S] document ids (pad = -1) -> int32 cu_seqlens over the flattened B*S axis and the longest segment.
    Padding tails become their own segments so that every row belongs to exactly one segment."""
    flat = document_ids.reshape(-1)
    S = document_ids.shape[-1]
    pos = torch.arange(flat.numel(), device=flat.device)
    change = torch.ones_like(flat, dtype=torch.bool)
    change[1:] = (flat[1:] != flat[:-1]) | (pos[1:] % S == 0)
    starts = pos[change]
    cu = torch.cat((starts, torch.tensor([flat.numel()], device=flat.device))).to(torch.int32)
    return cu, int((cu[1:] - cu[:-1]).max())


@reference_kwargs(max_seq_len="max_length")
def get_packing_stats(lengths: Sequence[int], max_length: int) -> dict:
    bins = first_fit_decreasing(lengths, max_length)
    used = sum(min(n, max_length) for n in lengths)
    return {"num_sequences": len(lengths), "num_packed": len(bins), "efficiency": used / max(1, len(bins) * max_length),
            "padding_efficiency": used / max(1, len(lengths) * max_length),
            "compression_ratio": len(lengths) / max(1, len(bins))}


def calculate_packing_efficiency(lengths: Sequence[int], bins: Sequence[Sequence[int]], max_capacity: int) -> float:
    """Used tokens / capacity of the bins (1.0 = no padding)."""
    total = len(bins) * max_capacity
    return sum(lengths) / total if total > 0 else 0.0
