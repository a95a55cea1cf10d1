"""Sharded checkpoints in the torch.distributed.checkpoint (DCP) directory format.

The reference writes its sharded FSDP checkpoints with ONE `dcp.save` of `{"model": ..., "optimizer": ...}` taken from
`get_state_dict` (data_pipeline/trainer/distributed/fsdp2.py:2287-2363) plus a `meta.pt` whose `api_version` is
"dcp_modern_v2", and reads them back with `dcp.load` (:2684-2730).  This module writes and reads the same directory
from the flat engine:

  <dir>/.metadata, <dir>/__<rank>_<n>.distcp     DCP storage (FileSystemWriter)
      model.<hf name>                            fp32 master weights under HuggingFace parameter names
      optimizer.state.<hf name>.exp_avg / exp_avg_sq / step
      optimizer.param_groups                     [{lr, betas, eps, weight_decay, params: [hf names]}]
  <dir>/meta.pt                                  {epoch, step, api_version: "dcp_modern_v2", config{...}, extra{...}}

The engine's shards cut a unit's flat buffer at arbitrary offsets, so parameters are first gathered unit by unit
(fp32 masters and both moments), renamed / split to the HuggingFace layout (q/k/v out of the fused qkv, gate/up out of
gate|up), and every whole tensor is then WRITTEN BY ONE RANK (round-robin), which keeps the files balanced and the
metadata free of engine-specific chunking: any DCP reader (the reference's `dcp_load` into an FSDP model of the same
architecture, or `dcp.load` into plain tensors) can re-shard it.  Loading goes the other way, one unit at a time.
Every function here is collective over the engine's process group.
"""
from __future__ import annotations

from pathlib import Path

import torch
import torch.distributed as dist

from ..core.errors import CheckpointLoadError, CheckpointSaveError

API_VERSION = "dcp_modern_v2"


# ------------------------------------------------------------------------------------------------ name mapping
def _split_rows(t: torch.Tensor, sizes):
    return list(t.split(list(sizes), dim=0))


def to_hf_items(name: str, t: torch.Tensor, cfg) -> list[tuple[str, torch.Tensor]]:
    """One tensor under this framework's parameter name -> [(HuggingFace name, tensor)] (views, no copies)."""
    D, Hq, Hkv, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    if name == "lm_head":
        return [("lm_head.weight", t)]
    if name.endswith("self_attn.wqkv"):
        base = name[:-len("wqkv")]
        q, k, v = _split_rows(t, (Hq * D, Hkv * D, Hkv * D))
        return [(base + "q_proj.weight", q), (base + "k_proj.weight", k), (base + "v_proj.weight", v)]
    if name.endswith("self_attn.bqkv"):
        base = name[:-len("bqkv")]
        q, k, v = _split_rows(t, (Hq * D, Hkv * D, Hkv * D))
        return [(base + "q_proj.bias", q), (base + "k_proj.bias", k), (base + "v_proj.bias", v)]
    if name.endswith("self_attn.wo"):
        return [(name[:-len("wo")] + "o_proj.weight", t)]
    if name.endswith("mlp.w_gate_up") and t.dim() == 2:
        base = name[:-len("w_gate_up")]
        g, u = _split_rows(t, (I, I))
        return [(base + "gate_proj.weight", g), (base + "up_proj.weight", u)]
    if name.endswith("mlp.w_down") and t.dim() == 2:
        return [(name[:-len("w_down")] + "down_proj.weight", t)]
    if name.endswith("mlp.router"):
        return [(name[:-len("router")] + "gate.weight", t)]
    if name.endswith("mlp.w_gate_up"):
        return [(name[:-len("w_gate_up")] + "experts.gate_up_proj", t)]
    if name.endswith("mlp.w_down"):
        return [(name[:-len("w_down")] + "experts.down_proj", t)]
    return [(name, t)]       # embeddings and norm weights already carry their HuggingFace names


def _unit_full(engine, u, shard: torch.Tensor) -> torch.Tensor:
    """All ranks' shards of one per-unit fp32 buffer, concatenated (on the engine's device)."""
    if engine.world == 1 or engine.cfg.sharding_strategy == "NO_SHARD":
        return shard
    full = torch.empty(u.numel, dtype=shard.dtype, device=shard.device)
    if shard.is_cuda:
        dist.all_gather_into_tensor(full, shard.contiguous(), group=engine.pg)
    else:
        parts = list(full.chunk(engine.world))
        dist.all_gather(parts, shard.contiguous(), group=engine.pg)
    return full


def _hf_entries(u, full: torch.Tensor, cfg) -> list[tuple[str, torch.Tensor]]:
    out = []
    for (n, p, o, k) in u.entries:
        out.extend(to_hf_items(n, full[o:o + k].view(p.shape), cfg))
    return out


# ------------------------------------------------------------------------------------------------ save
def save_dcp_checkpoint(engine, model, path, epoch: int = 0, step: int = 0, extra: dict | None = None) -> None:
    """Write the model (fp32 masters) and the AdamW state of a flat engine as a DCP directory (module docstring)."""
    import torch.distributed.checkpoint as dcp
    from . import atomic_torch_save
    path = Path(path)
    cfg = model.config
    rank, world = engine.rank, engine.world
    distributed = engine.distributed
    try:
        if rank == 0:
            path.mkdir(parents=True, exist_ok=True)
        if distributed:
            dist.barrier(group=engine.pg)
        state: dict = {"model": {}, "optimizer": {"state": {}}}
        names: list[str] = []
        idx = 0
        step_t = torch.tensor(float(engine.step_count))
        for u in engine.units:
            bufs = {"model": u.master, "exp_avg": u.exp_avg, "exp_avg_sq": u.exp_avg_sq}
            fulls = {k: (None if v is None else _unit_full(engine, u, v)) for k, v in bufs.items()}
            for hf, t in _hf_entries(u, fulls["model"], cfg):
                names.append(hf)
                mine = idx % world == rank
                idx += 1
                if not mine:
                    continue                      # another rank writes this tensor
                state["model"][hf] = t.detach().cpu().clone()
            for key in ("exp_avg", "exp_avg_sq"):
                if fulls[key] is None:
                    continue
                for j, (hf, t) in enumerate(_hf_entries(u, fulls[key], cfg)):
                    if (names.index(hf)) % world == rank:
                        state["optimizer"]["state"].setdefault(hf, {"step": step_t.clone()})[key] = \
                            t.detach().cpu().clone()
            del fulls
        if rank == 0:
            g = dict(engine.param_groups[0])
            g["betas"] = tuple(g.get("betas", ()))
            g["params"] = names
            state["optimizer"]["param_groups"] = [g]
        dcp.save(state, storage_writer=dcp.FileSystemWriter(str(path), overwrite=True),
                 process_group=engine.pg if distributed else None, no_dist=not distributed)
        if rank == 0:
            atomic_torch_save({"epoch": epoch, "step": step, "api_version": API_VERSION,
                               "config": {"sharding_strategy": engine.cfg.sharding_strategy,
                                          "mixed_precision": str(engine.cfg.param_dtype), "world_size": world},
                               "extra": extra or {}}, path / "meta.pt")
        if distributed:
            dist.barrier(group=engine.pg)
    except (OSError, RuntimeError) as e:
        raise CheckpointSaveError(f"failed to write DCP checkpoint {path}", cause=e)


# ------------------------------------------------------------------------------------------------ load
def is_dcp_checkpoint(path) -> bool:
    return (Path(path) / ".metadata").exists()


def load_dcp_checkpoint(engine, model, path, load_optimizer: bool = True) -> dict:
    """Read a DCP directory (written here or by the reference for a model with the same HuggingFace parameter names)
    into the engine: fp32 masters, bf16 parameters (cast from the masters), both AdamW moments and the step count.
    Works at any world size; returns the `meta.pt` dictionary ({} if absent)."""
    import torch.distributed.checkpoint as dcp
    path = Path(path)
    if not is_dcp_checkpoint(path):
        raise CheckpointLoadError(f"{path} has no .metadata file: not a torch.distributed.checkpoint directory")
    cfg = model.config
    distributed = engine.distributed
    reader = dcp.FileSystemReader(str(path))
    known = set(reader.read_metadata().state_dict_metadata.keys())
    try:
        step_seen = None
        engine.drop_gathered()
        for u in engine.units:
            for key, dst in (("model", u.master), ("exp_avg", u.exp_avg), ("exp_avg_sq", u.exp_avg_sq)):
                if dst is None or (key != "model" and not load_optimizer):
                    continue
                full = torch.zeros(u.numel, dtype=torch.float32)
                want: dict = {}
                for hf, view in _hf_entries(u, full, cfg):
                    fq = f"model.{hf}" if key == "model" else f"optimizer.state.{hf}.{key}"
                    if fq in known:
                        want[fq] = view        # DCP copies into this view of `full` in place
                if not want:
                    if key == "model":
                        raise CheckpointLoadError(f"unit {u.name}: none of its parameters is in {path}")
                    continue
                nested: dict = {}
                for fq, view in want.items():
                    cur = nested
                    parts = _split_fqn(fq)
                    for p_ in parts[:-1]:
                        cur = cur.setdefault(p_, {})
                    # non-contiguous row views (q / k / v inside the fused buffer) are contiguous here: row splits
                    cur[parts[-1]] = view
                dcp.load(nested, storage_reader=reader, process_group=engine.pg if distributed else None,
                         no_dist=not distributed)
                s0 = u.shard_start
                dst.copy_(full[s0:s0 + u.shard_numel])
                if key == "model":
                    tgt = u.param_shard if u.resharded else u.flat_param[s0:s0 + u.shard_numel]
                    tgt.copy_(dst)
            if load_optimizer and step_seen is None:
                for hf, _ in _hf_entries(u, torch.zeros(u.numel), cfg)[:1]:
                    fq = f"optimizer.state.{hf}.step"
                    if fq in known:
                        box = {"optimizer": {"state": {hf: {"step": torch.zeros(())}}}}
                        dcp.load(box, storage_reader=reader, process_group=engine.pg if distributed else None,
                                 no_dist=not distributed)
                        step_seen = int(box["optimizer"]["state"][hf]["step"].item())
        if step_seen is not None:
            engine.step_count = step_seen
        # the parameters every rank keeps gathered are rebuilt from the freshly loaded shards
        if engine.world > 1 and engine.cfg.sharding_strategy != "NO_SHARD":
            if engine.is_cuda:
                torch.cuda.synchronize(engine.device)
            dist.barrier(group=engine.pg)
            engine._all_gather_params()
            if engine._symm is not None:
                engine._device_barrier()
        meta_f = path / "meta.pt"
        return torch.load(meta_f, map_location="cpu", weights_only=False) if meta_f.exists() else {}
    except (OSError, RuntimeError, KeyError) as e:
        raise CheckpointLoadError(f"failed to load DCP checkpoint {path}", cause=e)


def _split_fqn(fq: str) -> list[str]:
    """'optimizer.state.<hf name with dots>.exp_avg' -> ['optimizer', 'state', '<hf name>', 'exp_avg']; DCP flattens
    nested dictionaries by joining keys with dots, and parameter names contain dots themselves."""
    if fq.startswith("model."):
        return ["model", fq[len("model."):]]
    if fq.startswith("optimizer.state."):
        rest = fq[len("optimizer.state."):]
        name, leaf = rest.rsplit(".", 1)
        return ["optimizer", "state", name, leaf]
    return fq.split(".")
