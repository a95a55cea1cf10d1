"""Synthetic token data: uniform-random ids of a fixed shape, optionally packed with document boundaries.

Every benchmark configuration trains on this (there is no dataset access on the benchmark machines): token ids
uniform in [0, vocab), document lengths ~ U(min_doc, max_doc) packed into fixed-length sequences, with the batch
schema of the real pipeline (input_ids / attention_mask / labels, plus position_ids / document_ids / cu_seqlens
for packed batches; preprocessing/prompt_engine.py:145-169 and trainer/packing.py:183-191 of the reference).
"""
from __future__ import annotations

import torch
from torch.utils.data import DataLoader, Dataset


class SyntheticTokenDataset(Dataset):
    def __init__(self, vocab_size: int, seq_len: int, num_samples: int = 1 << 16, seed: int = 0,
                 packed: bool = False, min_doc: int = 64, max_doc: int = 512, mode: str = "uniform"):
        self.mode = mode    # "uniform": i.i.d. tokens (benchmarks); "arith": t[i+1] = t[i] + 7 mod V (a learnable toy task)
        self.vocab_size, self.seq_len, self.num_samples, self.seed = vocab_size, seq_len, num_samples, seed
        self.packed, self.min_doc, self.max_doc = packed, min_doc, max_doc

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1000003 + idx)
        ids = torch.randint(0, self.vocab_size, (self.seq_len,), generator=g, dtype=torch.int64)
        if self.mode == "arith":
            ids = (ids[0] + 7 * torch.arange(self.seq_len)) % self.vocab_size
        item = {"input_ids": ids, "attention_mask": torch.ones(self.seq_len, dtype=torch.int64), "labels": ids.clone()}
        if self.packed:
            doc = torch.empty(self.seq_len, dtype=torch.int64)
            pos = torch.empty(self.seq_len, dtype=torch.int64)
            s, d = 0, 0
            while s < self.seq_len:
                n = int(torch.randint(self.min_doc, self.max_doc + 1, (1,), generator=g))
                e = min(self.seq_len, s + n)
                doc[s:e] = d
                pos[s:e] = torch.arange(e - s)
                s, d = e, d + 1
            item["document_ids"], item["position_ids"] = doc, pos
        return item


class SyntheticPreferenceDataset(Dataset):
    """prompt / chosen / rejected triples of fixed lengths (DPO-style batches)."""

    def __init__(self, vocab_size: int, prompt_len: int, response_len: int, num_samples: int = 1 << 14, seed: int = 0):
        self.v, self.p, self.r, self.n, self.seed = vocab_size, prompt_len, response_len, num_samples, seed

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 7919 + idx)
        prompt = torch.randint(0, self.v, (self.p,), generator=g)
        out = {}
        for name in ("chosen", "rejected"):
            resp = torch.randint(0, self.v, (self.r,), generator=g)
            ids = torch.cat((prompt, resp))
            labels = ids.clone()
            labels[: self.p] = -100
            out[f"{name}_input_ids"] = ids
            out[f"{name}_attention_mask"] = torch.ones_like(ids)
            out[f"{name}_labels"] = labels
        out["prompt_input_ids"] = prompt
        out["prompt_attention_mask"] = torch.ones_like(prompt)
        return out


def synthetic_dataloader(vocab_size: int, seq_len: int, batch_size: int, num_batches: int = 64, seed: int = 0,
                         packed: bool = False, pin_memory: bool = False, num_workers: int = 0, rank: int = 0,
                         **kw) -> DataLoader:
    ds = SyntheticTokenDataset(vocab_size, seq_len, num_batches * batch_size, seed * 977 + rank, packed, **kw)
    return DataLoader(ds, batch_size=batch_size, shuffle=False, drop_last=True, pin_memory=pin_memory,
                      num_workers=num_workers)


def synthetic_preference_dataloader(vocab_size: int, prompt_len: int, response_len: int, batch_size: int,
                                    num_batches: int = 64, seed: int = 0, pin_memory: bool = False, rank: int = 0,
                                    num_workers: int = 0) -> DataLoader:
    """Batches of prompt / chosen / rejected triples with the keys of the reference's preference stage
    (data_pipeline/preprocessing/prompt_engine.py:1896-1979): chosen_/rejected_ input_ids, attention_mask, labels
    (prompt positions masked with -100), prompt_input_ids, prompt_attention_mask."""
    ds = SyntheticPreferenceDataset(vocab_size, prompt_len, response_len, num_batches * batch_size, seed * 977 + rank)
    return DataLoader(ds, batch_size=batch_size, shuffle=False, drop_last=True, pin_memory=pin_memory,
                      num_workers=num_workers)
