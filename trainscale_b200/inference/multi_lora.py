"""Batched multi-adapter LoRA for the continuous-batching engine: tokens of requests that use DIFFERENT adapters run in
one step.

For every adapted weight the adapters are stored stacked, A [n, R, in] and B [n, out, R] (R = the sum of the ranks of
the weight's row blocks, zero-padded to a multiple of 64; the scaling is folded into B).  A token batch with per-token
adapter ids is sorted by adapter with the MoE routing plan (`ops/moe.py`: device-side ranks, 128-aligned segments) and
the two low-rank products run as grouped tcgen05 GEMMs - the same kernel that serves experts - followed by the
un-permute.  Tokens without an adapter go to a zero "null" adapter, so the batch never has to be split on the host.
On CPU (tests) the same maths runs as a loop over the adapters present.

The reference delegates multi-LoRA serving to vLLM (data_pipeline/trainer/inference.py:346-374 `LoRAConfig`:
max_loras, max_lora_rank); this is the in-framework equivalent.
"""
from __future__ import annotations

import torch

from ..ops import moe as _moe

PAD_RANK = 64        # grouped GEMM needs the reduction length to be a multiple of its K tile


class BatchedLoRA:
    """Adapters of one model (whose LoRA modules are attached by `lora.get_peft_model`), stacked for batched use."""

    def __init__(self, model, adapters: dict[str, dict[str, torch.Tensor]]):
        """`adapters`: name -> {parameter name: tensor} as produced by `lora.lora_state_dict` / the adapter registry."""
        self.names = list(adapters)
        self.index = {n: i for i, n in enumerate(self.names)}
        self.null = len(self.names)                      # id of the all-zero adapter
        E = self.null + 1
        dev = next(model.parameters()).device
        dt = next(model.parameters()).dtype
        self.weights: dict[tuple[int, str], tuple[torch.Tensor, torch.Tensor]] = {}
        for li, layer in enumerate(model.model.layers):
            for hf, mod in (("self_attn", layer.self_attn), ("mlp", layer.mlp)):
                inner = getattr(mod, "inner", mod)
                if getattr(inner, "lora", None) is None:
                    continue
                for wname, fused in inner.lora.items():
                    W = getattr(inner, wname)
                    R = sum(p.r for p in fused.parts)
                    Rp = (R + PAD_RANK - 1) // PAD_RANK * PAD_RANK
                    A = torch.zeros(E, Rp, W.shape[1], dtype=dt, device=dev)
                    B = torch.zeros(E, W.shape[0], Rp, dtype=dt, device=dev)
                    for ai, name in enumerate(self.names):
                        st, c0 = adapters[name], 0
                        for pi, p in enumerate(fused.parts):
                            key = f"model.layers.{li}.{hf}.lora.{wname}.parts.{pi}."
                            a, b = st[key + "lora_A"], st[key + "lora_B"]
                            A[ai, c0:c0 + p.r] = a.to(dev, dt)
                            B[ai, p.row0:p.row0 + p.rows, c0:c0 + p.r] = (b.float() * p.scaling).to(dev, dt)
                            c0 += p.r
                    self.weights[(li, wname)] = (A, B)

    def ids_for(self, names: list[str | None]) -> list[int]:
        return [self.null if n is None else self.index[n] for n in names]

    def delta(self, layer: int, wname: str, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor | None:
        """x [T, in], ids [T] (adapter index per token) -> [T, out] low-rank update, or None if nothing applies."""
        ab = self.weights.get((layer, wname))
        if ab is None:
            return None
        A, B = ab
        E = A.shape[0]
        if _moe.available(x):
            plan = _moe.make_plan(ids.view(-1, 1).to(torch.int32), E)
            xp = _moe._PermuteFn.apply(x, plan)
            y = _moe.grouped_linear(_moe.grouped_linear(xp, A, plan), B, plan)
            ones = torch.ones(x.shape[0], 1, dtype=x.dtype, device=x.device)
            return _moe._CombineFn.apply(y, ones, plan)
        out = torch.zeros(x.shape[0], B.shape[1], dtype=x.dtype, device=x.device)
        for a in ids.unique().tolist():
            if a == self.null:
                continue
            sel = (ids == a).nonzero(as_tuple=True)[0]
            out[sel] = ((x[sel].float() @ A[a].float().t()) @ B[a].float().t()).to(x.dtype)
        return out
