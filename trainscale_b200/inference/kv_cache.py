"""Paged KV cache: fixed-size blocks, per-sequence block tables, prefix sharing by reference counts."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import torch


class BlockAllocator:
    """Reference-counted blocks. A released block whose content is indexed by a prefix hash stays reusable (it moves
    to an LRU pool and is only overwritten when no plain free block is left)."""

    def __init__(self, num_blocks: int):
        from collections import OrderedDict
        self.num_blocks = num_blocks
        self.free = list(range(num_blocks - 1, -1, -1))
        self.free_cached: "OrderedDict[int, None]" = OrderedDict()
        self.ref = [0] * num_blocks
        self.prefix_index: dict[bytes, int] = {}     # hash of a full block's tokens (+ parent hash) -> block id
        self.block_hash: dict[int, bytes] = {}

    @property
    def num_free(self) -> int:
        return len(self.free) + len(self.free_cached)

    def allocate(self) -> int:
        if self.free:
            b = self.free.pop()
        elif self.free_cached:
            b, _ = self.free_cached.popitem(last=False)      # evict the least recently released cached block
            h = self.block_hash.pop(b, None)
            if h is not None and self.prefix_index.get(h) == b:
                del self.prefix_index[h]
        else:
            raise MemoryError("KV cache is out of blocks")
        self.ref[b] = 1
        return b

    def share(self, b: int) -> int:
        if self.ref[b] == 0:
            self.free_cached.pop(b, None)
        self.ref[b] += 1
        return b

    def release(self, b: int) -> None:
        self.ref[b] -= 1
        if self.ref[b] == 0:
            if b in self.block_hash:
                self.free_cached[b] = None
            else:
                self.free.append(b)


@dataclass
class SequenceBlocks:
    blocks: list[int] = field(default_factory=list)
    num_tokens: int = 0


class PagedKVCache:
    """k/v caches [layers][num_blocks, block_size, Hkv, D]."""

    def __init__(self, num_layers: int, num_blocks: int, block_size: int, n_kv_heads: int, head_dim: int, dtype, device,
                 enable_prefix_caching: bool = True):
        self.block_size, self.num_layers = block_size, num_layers
        self.alloc = BlockAllocator(num_blocks)
        # one block beyond the allocator's range: padding rows of a fixed-shape (CUDA-graph) decode batch write their
        # key / value there and read it back as their one-token "sequence"
        self.trash_block = num_blocks
        shape = (num_blocks + 1, block_size, n_kv_heads, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.seqs: dict[int, SequenceBlocks] = {}
        self.prefix_caching = enable_prefix_caching
        self.prefix_hits = 0

    def blocks_needed(self, seq_id: int, new_tokens: int) -> int:
        s = self.seqs.get(seq_id)
        have = len(s.blocks) * self.block_size if s else 0
        used = s.num_tokens if s else 0
        return max(0, -(-(used + new_tokens - have) // self.block_size))

    def can_append(self, seq_id: int, new_tokens: int) -> bool:
        return self.blocks_needed(seq_id, new_tokens) <= self.alloc.num_free

    def match_prefix(self, seq_id: int, tokens: list[int], salt: bytes = b"") -> int:
        """Reuse cached full blocks that hold the same token prefix; returns the number of tokens covered.
        `salt` separates caches whose keys / values differ for the same tokens (e.g. another LoRA adapter)."""
        s = self.seqs.setdefault(seq_id, SequenceBlocks())
        if not self.prefix_caching or s.blocks:
            return 0
        parent = salt
        covered = 0
        # never cover the whole prompt: at least one token must run through the model to produce logits
        for i in range(0, max(0, len(tokens) - 1) // self.block_size * self.block_size, self.block_size):
            h = hashlib.sha1(parent + str(tokens[i:i + self.block_size]).encode()).digest()
            b = self.alloc.prefix_index.get(h)
            if b is None:
                break
            s.blocks.append(self.alloc.share(b))
            covered += self.block_size
            parent = h
        s.num_tokens = covered
        if covered:
            self.prefix_hits += covered
        return covered

    def append_slots(self, seq_id: int, n: int) -> list[int]:
        """Reserve n token slots at the end of the sequence; returns flat slot ids (block * block_size + offset)."""
        s = self.seqs.setdefault(seq_id, SequenceBlocks())
        slots = []
        for _ in range(n):
            if s.num_tokens == len(s.blocks) * self.block_size:
                s.blocks.append(self.alloc.allocate())
            b = s.blocks[s.num_tokens // self.block_size]
            slots.append(b * self.block_size + s.num_tokens % self.block_size)
            s.num_tokens += 1
        return slots

    def register_full_blocks(self, seq_id: int, tokens: list[int], salt: bytes = b"") -> None:
        if not self.prefix_caching:
            return
        s = self.seqs[seq_id]
        parent = salt
        for bi in range(min(len(s.blocks), len(tokens) // self.block_size)):
            h = hashlib.sha1(parent + str(tokens[bi * self.block_size:(bi + 1) * self.block_size]).encode()).digest()
            b = s.blocks[bi]
            if h not in self.alloc.prefix_index:
                self.alloc.prefix_index[h] = b
                self.alloc.block_hash[b] = h
            parent = h

    def free_sequence(self, seq_id: int) -> None:
        s = self.seqs.pop(seq_id, None)
        if s:
            for b in s.blocks:
                self.alloc.release(b)

    def block_table(self, seq_ids: list[int], device) -> tuple[torch.Tensor, torch.Tensor]:
        mx = max((len(self.seqs[i].blocks) for i in seq_ids), default=1)
        bt = torch.zeros(len(seq_ids), max(mx, 1), dtype=torch.int32)
        for r, i in enumerate(seq_ids):
            b = self.seqs[i].blocks
            bt[r, :len(b)] = torch.tensor(b, dtype=torch.int32)
        lens = torch.tensor([self.seqs[i].num_tokens for i in seq_ids], dtype=torch.int32)
        if device is None:
            return bt, lens
        return bt.to(device), lens.to(device)

    def utilization(self) -> float:
        return 1.0 - self.alloc.num_free / self.alloc.num_blocks
