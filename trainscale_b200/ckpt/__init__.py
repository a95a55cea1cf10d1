"""Checkpoint save / resume.

Directory layout follows data_pipeline/trainer/trainers/sota_trainer.py:2920-3314 and
data_pipeline/trainer/distributed/fsdp2.py:2317-2363:

  checkpoint-{step}/
    model.safetensors (+ config.json)   full weights in HuggingFace Llama naming, written by rank 0
    optim/shard-{rank:05d}-of-{world:05d}.pt   this rank's fp32 master / moment slices (flat engine)
      -- or, with `distributed.fsdp_config.checkpoint_format: dcp`, instead of the two entries above --
    .metadata + __{rank}_{n}.distcp     torch.distributed.checkpoint directory (ckpt/dcp.py): fp32 weights and AdamW
                                        state under HuggingFace parameter names, the reference's `dcp_save` layout
    meta.pt            {epoch, step, api_version, config{sharding_strategy, mixed_precision, world_size}, extra{...}}
    trainer_state.pt   {optimizer|None, scheduler, state{...}, config, rng_state{python,numpy,torch,cuda}, meta{...}}

Every file is written to `<name>.tmp` and renamed, tensors are moved to CPU first, and a world-size mismatch on
resume re-slices the flat optimizer shards instead of failing (`reshard_optimizer_state`).
"""
from __future__ import annotations

import contextlib

import json
import os
import time
from dataclasses import asdict
from pathlib import Path

import torch
import torch.distributed as dist

from ..core.errors import CheckpointLoadError, CheckpointSaveError

API_VERSION = "ts_flat_v1"


def atomic_torch_save(obj, path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + ".tmp")
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _to_cpu(o):
    if torch.is_tensor(o):
        return o.detach().cpu()
    if isinstance(o, dict):
        return {k: _to_cpu(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(_to_cpu(v) for v in o)
    return o


def save_model_weights(model, path: Path, max_shard_bytes: int = 5 * 2 ** 30) -> None:
    """HF-format weights: safetensors shards + index (or model.pt when safetensors is unavailable)."""
    from ..hub import ModelSerializer
    sd = model.to_hf_state_dict() if hasattr(model, "to_hf_state_dict") else model.state_dict()
    ModelSerializer(max_shard_bytes).save(sd, path)
    if hasattr(model, "hf_config_dict"):
        (path / "config.json").write_text(json.dumps(model.hf_config_dict(), indent=2))


def save_model_parallel_weights(trainer, path: Path) -> None:
    """Weights of a tensor- / pipeline-parallel run as ONE HuggingFace-layout checkpoint.  Every tensor-parallel
    group gathers its projections to full width; the ranks whose tp / dp / cp coordinates are 0 (one per pipeline
    stage) write their stage's layers as shard files of a common numbering, and global rank 0 writes the index over
    all stages.  Collective: every rank calls it."""
    from ..hub import HAVE_SAFETENSORS, ModelSerializer
    eng, model = trainer.engine, trainer.model
    dims = eng.dims
    first = last = True
    if eng.pipelined:
        first, last = eng.stage_module.first, eng.stage_module.last
    writer = dims.local_rank("tp") == 0 and dims.local_rank("dp_cp") == 0
    sd = model.to_hf_state_dict(tp=eng.tp, first=first, last=last, keep=writer)
    if not writer:
        return
    P, stage = dims.size("pp"), dims.pp_stage
    if P > 1 and not HAVE_SAFETENSORS:
        raise CheckpointSaveError("a pipelined checkpoint needs the safetensors package (one shard file per stage)")
    ser = ModelSerializer()
    if P == 1:
        ser.save(sd, path)
    else:
        counts = [None] * P
        dist.all_gather_object(counts, len(ser.plan(sd)), group=dims.group("pp"))
        part = ser.save_part(sd, path, sum(counts[:stage]), sum(counts))
        parts = [None] * P
        dist.all_gather_object(parts, part, group=dims.group("pp"))
        if stage == 0:
            ser.write_index(path, parts)
    if trainer.rank == 0 and hasattr(model, "hf_config_dict"):
        (path / "config.json").write_text(json.dumps(model.hf_config_dict(), indent=2))


def load_model_weights(model, path: Path, strict: bool = True, tp=None) -> None:
    from ..hub import ModelDeserializer
    sd = ModelDeserializer().load(path)
    if tp is not None:
        model.load_hf_state_dict(sd, strict=strict, tp=tp)
    elif hasattr(model, "load_hf_state_dict"):
        model.load_hf_state_dict(sd, strict=strict)
    else:
        model.load_state_dict(sd, strict=strict)


def save_training_checkpoint(trainer, path: Path) -> None:
    path = Path(path)
    rank, world = trainer.rank, trainer.world_size
    try:
        if trainer.is_distributed:
            dist.barrier()
        eng = trainer.engine
        fmt = str((trainer.config.distributed.fsdp_config or {}).get("checkpoint_format", "")).lower()
        if fmt == "dcp" and eng is not None and hasattr(eng, "units") and not hasattr(eng, "dims") \
                and hasattr(trainer.model, "config"):
            from .dcp import save_dcp_checkpoint
            st = trainer.state
            save_dcp_checkpoint(eng, trainer.model, path, st.epoch, st.global_step,
                                {"best_metric": st.best_metric, "patience_counter": st.patience_counter,
                                 "samples_seen": st.samples_seen})
            if rank == 0:
                _save_trainer_state(trainer, path, None, world, rank)
                if hasattr(trainer.model, "hf_config_dict"):
                    (path / "config.json").write_text(json.dumps(trainer.model.hf_config_dict(), indent=2))
            if trainer.is_distributed:
                dist.barrier()
            return
        # FULL_SHARD keeps only shards between steps: every rank takes part in materialising the weights
        summon = eng.summon_full_params() if eng is not None and hasattr(eng, "summon_full_params") \
            else contextlib.nullcontext()
        with summon:
            if rank == 0:
                path.mkdir(parents=True, exist_ok=True)
            if eng is not None and hasattr(eng, "dims") and (eng.tp is not None or eng.pipelined):
                if trainer.is_distributed:
                    dist.barrier()
                save_model_parallel_weights(trainer, path)
            elif eng is not None and hasattr(eng, "ep_group"):
                # expert parallelism: every rank takes part in gathering the experts, rank 0 writes
                from ..hub import ModelSerializer
                sd = trainer.model.to_hf_state_dict()
                if rank == 0:
                    ModelSerializer().save(sd, path)
                    (path / "config.json").write_text(json.dumps(trainer.model.hf_config_dict(), indent=2))
                del sd
            elif rank == 0:
                save_model_weights(trainer.model, path)
        if trainer.is_distributed:
            dist.barrier()
        sharded = eng is not None and hasattr(eng, "state_dict")
        if sharded:
            write_shard = eng.cfg.sharding_strategy != "NO_SHARD" or rank == 0 if hasattr(eng, "cfg") else True
            if write_shard:
                atomic_torch_save(_to_cpu(eng.state_dict()), path / "optim" / f"shard-{rank:05d}-of-{world:05d}.pt")
        if rank == 0:
            st = trainer.state
            meta = {"epoch": st.epoch, "step": st.global_step, "api_version": API_VERSION,
                    "config": {"sharding_strategy": getattr(getattr(eng, "cfg", None), "sharding_strategy", "NONE"),
                               "mixed_precision": str(trainer.dtype), "world_size": world},
                    "extra": {"best_metric": st.best_metric, "patience_counter": st.patience_counter,
                              "samples_seen": st.samples_seen}}
            atomic_torch_save(meta, path / "meta.pt")
            opt_sd = None
            if not sharded and trainer.optimizer is not None and hasattr(trainer.optimizer, "state_dict"):
                opt_sd = _to_cpu(trainer.optimizer.state_dict())
            _save_trainer_state(trainer, path, opt_sd, world, rank)
        if trainer.is_distributed:
            dist.barrier()
    except OSError as e:
        raise CheckpointSaveError(f"failed to write checkpoint {path}", cause=e)


def _save_trainer_state(trainer, path: Path, opt_sd, world: int, rank: int) -> None:
    st = trainer.state
    ts = {"optimizer": opt_sd,
          "scheduler": trainer.scheduler.state_dict() if trainer.scheduler is not None else None,
          "state": asdict(st), "config": trainer.config.to_dict(), "rng_state": trainer._collect_rng_states(),
          "scaler": None,
          "meta": {"torch_version": torch.__version__, "world_size": world, "rank": rank,
                   "distributed_strategy": trainer.strategy, "timestamp": time.time()}}
    atomic_torch_save(ts, path / "trainer_state.pt")


def reshard_optimizer_state(shards: list[dict], new_rank: int, new_world: int,
                            layout: dict[str, tuple[int, int, int]] | None = None) -> dict:
    """Re-slice flat optimizer shards saved at one world size for another.

    A unit's flat buffer is padded to a multiple that depends on the world size, so the padded length at the new size
    can differ from the saved one.  `layout` (unit name -> (padded numel, shard start, shard numel) of the engine that
    will load the result; `engine_layout(engine)`) makes the slices exact; the padding holds zeros either way.
    Without it the saved padded length must divide by the new world size."""
    shards = sorted(shards, key=lambda s: s["rank"])
    out = {k: v for k, v in shards[0].items() if k != "units"}
    out.update(rank=new_rank, world=new_world, units={})
    for name in shards[0]["units"]:
        numel = shards[0]["units"][name]["numel"]
        full = {}
        for key in ("master", "exp_avg", "exp_avg_sq"):
            if shards[0]["units"][name][key] is None:
                full[key] = None
                continue
            full[key] = torch.cat([s["units"][name][key] for s in shards])[:numel]
        if layout is not None:
            new_numel, start, n_new = layout[name]
            for key, v in full.items():
                if v is not None and v.numel() < new_numel:
                    full[key] = torch.cat((v, v.new_zeros(new_numel - v.numel())))
            sl = slice(start, start + n_new)
            numel = new_numel
        else:
            n_new = numel // new_world
            if numel % new_world:
                raise CheckpointLoadError(f"unit {name}: {numel} elements do not divide over {new_world} ranks")
            start = new_rank * n_new
            sl = slice(start, start + n_new)
        out["units"][name] = {k: (None if v is None else v[sl].clone()) for k, v in full.items()}
        out["units"][name].update(shard_start=start, numel=numel)
    return out


def select_model_parallel_shards(shards: list[dict], mesh: dict) -> list[dict]:
    """Of the optimizer shards of a tensor- / pipeline-parallel run, those that hold the SAME parameters as the rank
    whose mesh coordinates are `mesh` ({axis: [rank, size]}, `NDEngine.mesh_coordinates`): equal tp and pp
    coordinates.  They form one data-parallel group and can be re-sliced among themselves; shards of another tp rank
    or pipeline stage hold other parameters under the same unit names and must never be concatenated with them.
    A checkpoint whose tp or pp size differs from the running layout, or whose shards carry no coordinates, is
    refused."""
    if any("mesh" not in s for s in shards):
        raise CheckpointLoadError("optimizer shards of this checkpoint carry no mesh coordinates: they can only be "
                                  "resumed at the world size and parallel layout they were written at")
    saved = shards[0]["mesh"]
    for axis in ("tp", "pp"):
        if int(saved[axis][1]) != int(mesh[axis][1]):
            raise CheckpointLoadError(f"the checkpoint was written with {axis}={saved[axis][1]}, this run uses "
                                      f"{axis}={mesh[axis][1]}: optimizer shards are re-sliced along the data-parallel "
                                      f"axis only; load the weights alone or resume with the saved {axis} size")
    mine = [s for s in shards if all(int(s["mesh"][a][0]) == int(mesh[a][0]) for a in ("tp", "pp"))]
    want = int(saved["dp_cp"][1])
    if len(mine) != want:
        raise CheckpointLoadError(f"found {len(mine)} optimizer shards for tp rank {mesh['tp'][0]}, pp stage "
                                  f"{mesh['pp'][0]}; the checkpoint was written by {want} data-parallel ranks")
    return sorted(mine, key=lambda s: int(s["mesh"]["dp_cp"][0]))


def engine_layout(engine) -> dict[str, tuple[int, int, int]]:
    return {u.name: (u.numel, u.shard_start, u.shard_numel) for u in engine.units}


def load_training_checkpoint(trainer, path: Path) -> None:
    path = Path(path)
    if not path.exists():
        raise CheckpointLoadError(f"checkpoint {path} does not exist")
    try:
        eng = trainer.engine
        from .dcp import is_dcp_checkpoint, load_dcp_checkpoint
        dcp_dir = is_dcp_checkpoint(path) and eng is not None and hasattr(eng, "units") and not hasattr(eng, "dims")
        if dcp_dir:
            load_dcp_checkpoint(eng, trainer.model, path)
        summon = eng.summon_full_params() if eng is not None and hasattr(eng, "summon_full_params") \
            else contextlib.nullcontext()
        with summon if not dcp_dir else contextlib.nullcontext():
            if dcp_dir:
                pass
            else:
                load_model_weights(trainer.model, path, strict=False, tp=getattr(eng, "tp", None))
            if eng is not None and hasattr(eng, "units") and not dcp_dir:
                # the flat buffers alias the parameters: refresh the shards and fp32 masters from the loaded weights
                for u in eng.units:
                    src = u.flat_param[u.shard_start:u.shard_start + u.shard_numel]
                    if getattr(u, "resharded", False):
                        u.param_shard.copy_(src)
                    u.master.copy_(src)
        if eng is not None and hasattr(eng, "units") and not dcp_dir:
            files = sorted((path / "optim").glob("shard-*.pt")) if (path / "optim").exists() else []
            if files:
                saved_world = int(files[0].stem.split("-of-")[1])
                mine = path / "optim" / f"shard-{trainer.rank:05d}-of-{trainer.world_size:05d}.pt"
                if saved_world == trainer.world_size and mine.exists():
                    sd = torch.load(mine, map_location="cpu", weights_only=False)
                    if hasattr(eng, "mesh_coordinates") and "mesh" in sd and \
                            {k: list(v) for k, v in sd["mesh"].items()} != eng.mesh_coordinates():
                        raise CheckpointLoadError(f"the checkpoint's parallel layout {sd['mesh']} differs from this "
                                                  f"run's {eng.mesh_coordinates()} at the same world size")
                    eng.load_state_dict(sd)
                elif hasattr(eng, "ep_group"):
                    raise CheckpointLoadError("optimizer shards of an expert-parallel run can only be resumed at the "
                                              f"world size they were written at ({saved_world})")
                elif hasattr(eng, "mesh_coordinates"):
                    shards = select_model_parallel_shards(
                        [torch.load(f, map_location="cpu", weights_only=False) for f in files], eng.mesh_coordinates())
                    flat = eng.flat
                    eng.load_state_dict(reshard_optimizer_state(shards, flat.rank, flat.world, engine_layout(eng)))
                elif eng.cfg.sharding_strategy == "NO_SHARD" and saved_world == trainer.world_size:
                    eng.load_state_dict(torch.load(files[0], map_location="cpu", weights_only=False))
                else:
                    shards = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
                    eng.load_state_dict(reshard_optimizer_state(shards, trainer.rank if eng.cfg.sharding_strategy != "NO_SHARD" else 0,
                                                                trainer.world_size if eng.cfg.sharding_strategy != "NO_SHARD" else 1,
                                                                engine_layout(eng)))
        tsf = path / "trainer_state.pt"
        if tsf.exists():
            ts = torch.load(tsf, map_location="cpu", weights_only=False)
            for k, v in ts.get("state", {}).items():
                if hasattr(trainer.state, k):
                    setattr(trainer.state, k, v)
            if ts.get("scheduler") is not None and trainer.scheduler is not None:
                trainer.scheduler.load_state_dict(ts["scheduler"])
            if ts.get("optimizer") is not None and trainer.optimizer is not None and eng is None:
                trainer.optimizer.load_state_dict(ts["optimizer"])
            if ts.get("rng_state") and ts.get("meta", {}).get("world_size") == trainer.world_size:
                trainer._restore_rng_states(ts["rng_state"])
    except CheckpointLoadError:
        raise
    except (OSError, KeyError, RuntimeError) as e:
        raise CheckpointLoadError(f"failed to load checkpoint {path}", cause=e)


# ------------------------------------------------------------------------------------------------ integrity / restart
def verify_checkpoint(path: Path, world_size: int | None = None) -> list[str]:
    """Problems of a checkpoint directory (empty list = usable): missing or unreadable metadata, weight shards whose
    sha256 differs from the index, missing / truncated optimizer shards.  Reads files only; no process group needed."""
    import zipfile
    from ..hub import compute_sha256
    path = Path(path)
    problems: list[str] = []
    if not path.is_dir():
        return [f"{path} is not a directory"]
    for name in ("meta.pt", "trainer_state.pt"):
        f = path / name
        if not f.exists():
            problems.append(f"{name} is missing (the save did not finish)")
            continue
        try:
            torch.load(f, map_location="cpu", weights_only=False)
        except Exception as e:   # noqa: BLE001 - any unpickling / zip error means the file is damaged
            problems.append(f"{name} is unreadable: {type(e).__name__}")
    idx = path / "model.safetensors.index.json"
    if idx.exists():
        try:
            index = json.loads(idx.read_text())
            hashes = index.get("metadata", {}).get("sha256", {})
            for name in sorted(set(index.get("weight_map", {}).values())):
                f = path / name
                if not f.exists():
                    problems.append(f"weight shard {name} is missing")
                elif name in hashes and compute_sha256(f) != hashes[name]:
                    problems.append(f"weight shard {name} does not match its sha256")
        except (OSError, ValueError) as e:
            problems.append(f"weight index is unreadable: {e}")
    elif (path / ".metadata").exists():
        if not list(path.glob("*.distcp")):
            problems.append("torch.distributed.checkpoint metadata without any .distcp data file")
    elif not (path / "model.safetensors").exists() and not (path / "model.pt").exists():
        problems.append("no model weights")
    shards = sorted((path / "optim").glob("shard-*.pt")) if (path / "optim").exists() else []
    if shards:
        saved_world = int(shards[0].stem.split("-of-")[1])
        have = {int(f.stem.split("-")[1]) for f in shards}
        strategy = None
        try:
            strategy = torch.load(path / "meta.pt", map_location="cpu", weights_only=False)["config"]["sharding_strategy"]
        except Exception:   # noqa: BLE001
            pass
        if strategy != "NO_SHARD" and have != set(range(saved_world)):
            problems.append(f"optimizer shards {sorted(set(range(saved_world)) - have)} of {saved_world} are missing")
        for f in shards:
            if not zipfile.is_zipfile(f):
                problems.append(f"optimizer shard {f.name} is truncated or corrupt")
    return problems


def list_checkpoints(output_dir: Path) -> list[Path]:
    """`checkpoint-<step>` directories of a run, oldest first."""
    out = []
    for d in Path(output_dir).glob("checkpoint-*"):
        try:
            out.append((int(d.name.split("-", 1)[1]), d))
        except ValueError:
            continue
    return [d for _, d in sorted(out)]


def find_latest_valid_checkpoint(output_dir: Path, log=None) -> Path | None:
    """Newest checkpoint that passes `verify_checkpoint`; damaged or half-written ones are skipped (and reported).
    This is what a restarted job (torchrun --max-restarts, or a fresh launch with another world size) resumes from."""
    for d in reversed(list_checkpoints(output_dir)):
        problems = verify_checkpoint(d)
        if not problems:
            return d
        if log is not None:
            log(f"skipping {d.name}: " + "; ".join(problems))
    return None
