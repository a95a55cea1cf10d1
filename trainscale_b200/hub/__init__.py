"""Model serialisation (sharded safetensors + index with sha256), local "hub" loading, retry / circuit-breaker
helpers and the checkpoint manager.

Surface after data_pipeline/trainer/hub/__init__.py:284-1652 (CircuitBreaker, RetryPolicy, execute_with_retry,
compute_sha256, ModelSerializer, ModelDeserializer, HubManager, generate_model_card, CheckpointManager).
Network pushes are delegated to `huggingface_hub` when it is importable and a token is configured.
"""
from __future__ import annotations

import hashlib
import json
import os
import random
import shutil
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable

import torch

from ..core.errors import CheckpointLoadError, HubError
from ..utils.refargs import ANY, reference_kwargs

try:
    from safetensors.torch import load_file as _st_load, save_file as _st_save
    HAVE_SAFETENSORS = True
except Exception:   # pragma: no cover
    HAVE_SAFETENSORS = False


class CircuitBreaker:
    """closed -> open after `failure_threshold` consecutive failures -> half-open after `reset_timeout` s."""

    def __init__(self, failure_threshold: int = 5, reset_timeout: float = 60.0, clock: Callable[[], float] = time.monotonic):
        self.failure_threshold, self.reset_timeout, self.clock = failure_threshold, reset_timeout, clock
        self.failures, self.opened_at, self.state = 0, None, "closed"

    def allow(self) -> bool:
        if self.state == "open" and self.clock() - self.opened_at >= self.reset_timeout:
            self.state = "half_open"
        return self.state != "open"

    def can_execute(self):
        """`allow()` as a Result: Ok(True), or Err(HubError with code CIRCUIT_OPEN and the seconds left to wait)."""
        from ..core.types import Err, Ok
        if self.allow():
            return Ok(True)
        left = self.reset_timeout - (self.clock() - self.opened_at)
        return Err(HubError(f"circuit open, retry after {left:.1f}s", code=HubErrorCode.CIRCUIT_OPEN,
                            failures=self.failures, retry_after_s=left))

    def record_success(self):
        self.failures, self.state, self.opened_at = 0, "closed", None

    def record_failure(self):
        self.failures += 1
        if self.state == "half_open" or self.failures >= self.failure_threshold:
            self.state, self.opened_at = "open", self.clock()


@dataclass
class RetryPolicy:
    max_attempts: int = 3
    base_delay: float = 0.5
    max_delay: float = 30.0
    backoff: float = 2.0
    jitter: float = 0.1
    retry_on: tuple = (OSError, TimeoutError, ConnectionError)

    def delay(self, attempt: int) -> float:
        d = min(self.max_delay, self.base_delay * self.backoff ** attempt)
        return d * (1.0 + random.uniform(-self.jitter, self.jitter))

    def compute_delay_ms(self, attempt: int) -> int:
        """`delay(attempt)` in whole milliseconds (attempt is 0-based)."""
        return int(round(self.delay(attempt) * 1e3))


@reference_kwargs({"metrics": ANY}, circuit="breaker")
def execute_with_retry(fn: Callable, policy: RetryPolicy | None = None, breaker: CircuitBreaker | None = None,
                       sleep: Callable[[float], None] = time.sleep):
    policy = policy or RetryPolicy()
    last = None
    for attempt in range(policy.max_attempts):
        if breaker is not None and not breaker.allow():
            raise HubError("circuit breaker is open", failures=breaker.failures)
        try:
            out = fn()
            if breaker is not None:
                breaker.record_success()
            return out
        except policy.retry_on as e:
            last = e
            if breaker is not None:
                breaker.record_failure()
            if attempt + 1 < policy.max_attempts:
                sleep(policy.delay(attempt))
    raise HubError(f"operation failed after {policy.max_attempts} attempts", cause=last)


@reference_kwargs(chunk_size="chunk")
def compute_sha256(path: str | os.PathLike, chunk: int = 1 << 22) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


class ModelSerializer:
    """state dict -> `model.safetensors` or `model-0000i-of-0000n.safetensors` + `model.safetensors.index.json`."""

    @reference_kwargs(shard_size_bytes="max_shard_bytes")
    def __init__(self, max_shard_bytes: int = 5 * 2 ** 30, prefer_safetensors: bool = True):
        if max_shard_bytes <= 0:
            raise ValueError("max_shard_bytes must be positive")
        self.max_shard_bytes, self.prefer_safetensors = max_shard_bytes, prefer_safetensors

    @property
    def shard_size_bytes(self) -> int:
        return self.max_shard_bytes

    @property
    def safetensors_available(self) -> bool:
        return HAVE_SAFETENSORS

    def serialize(self, model, output_dir: str | os.PathLike, model_id: str | None = None):
        """`model.state_dict()` written under `output_dir`; Ok(SerializationResult) or Err(HubError)
        (data_pipeline/trainer/hub/__init__.py:522-567)."""
        from ..core.types import Err, Ok
        try:
            self.save(model.state_dict(), output_dir)
            return Ok(SerializationResult.describe(output_dir))
        except Exception as e:   # noqa: BLE001
            return Err(HubError(f"failed to serialise model: {e}", code=HubErrorCode.SERIALIZATION_ERROR,
                                model_id=model_id, output_dir=str(output_dir)))

    def plan(self, sd: dict[str, torch.Tensor]) -> list[list[str]]:
        shards, cur, size = [], [], 0
        for k, v in sd.items():
            b = v.numel() * v.element_size()
            if cur and size + b > self.max_shard_bytes:
                shards.append(cur)
                cur, size = [], 0
            cur.append(k)
            size += b
        if cur:
            shards.append(cur)
        return shards

    def save(self, sd: dict[str, torch.Tensor], out_dir: str | os.PathLike) -> dict:
        out = Path(out_dir)
        out.mkdir(parents=True, exist_ok=True)
        if not (HAVE_SAFETENSORS and getattr(self, "prefer_safetensors", True)):
            sd = {k: v.detach().cpu().contiguous() for k, v in sd.items()}
            tmp = out / "model.pt.tmp"
            torch.save(sd, tmp)
            os.replace(tmp, out / "model.pt")
            return {"format": "pt", "files": ["model.pt"]}
        part = self.save_part(sd, out, 0, len(self.plan(sd)))
        self.write_index(out, [part])
        return {"format": "safetensors", "files": part["files"]}

    def save_part(self, sd: dict[str, torch.Tensor], out_dir: str | os.PathLike, first_index: int, total: int) -> dict:
        """Write this writer's tensors as shard files number first_index+1 ... of `total` (several writers, e.g. one
        per pipeline stage, fill one directory); returns {files, weight_map, sha256, total_size} for `write_index`."""
        out = Path(out_dir)
        out.mkdir(parents=True, exist_ok=True)
        sd = {k: v.detach().cpu().contiguous() for k, v in sd.items()}
        # tied tensors share storage: safetensors refuses aliases, so clone duplicates
        seen: dict[int, str] = {}
        for k, v in list(sd.items()):
            p = v.data_ptr()
            if p in seen and v.numel() > 0:
                sd[k] = v.clone()
            seen[p] = k
        weight_map, files, hashes = {}, [], {}
        for i, keys in enumerate(self.plan(sd)):
            name = "model.safetensors" if total == 1 else f"model-{first_index + i + 1:05d}-of-{total:05d}.safetensors"
            tmp = out / (name + ".tmp")
            _st_save({k: sd[k] for k in keys}, str(tmp), metadata={"format": "pt"})
            os.replace(tmp, out / name)
            files.append(name)
            hashes[name] = compute_sha256(out / name)
            weight_map.update({k: name for k in keys})
        return {"files": files, "weight_map": weight_map, "sha256": hashes,
                "total_size": sum(v.numel() * v.element_size() for v in sd.values())}

    @staticmethod
    def write_index(out_dir: str | os.PathLike, parts: list[dict]) -> None:
        weight_map, hashes, size = {}, {}, 0
        for p in parts:
            weight_map.update(p["weight_map"])
            hashes.update(p["sha256"])
            size += p["total_size"]
        index = {"metadata": {"total_size": size, "sha256": hashes}, "weight_map": weight_map}
        (Path(out_dir) / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))


class ModelDeserializer:
    @reference_kwargs(num_workers="num_threads")
    def __init__(self, verify_integrity: bool = True, num_threads: int = 4):
        self.verify, self.num_threads = verify_integrity, num_threads

    @reference_kwargs(model_dir="in_dir")
    def load(self, in_dir: str | os.PathLike, device=None) -> dict[str, torch.Tensor]:
        """State dict of the folder; `device` moves the tensors there (they are read on the host)."""
        sd = self._load(in_dir)
        return sd if device is None else {k: v.to(device) for k, v in sd.items()}

    def _load(self, in_dir: str | os.PathLike) -> dict[str, torch.Tensor]:
        d = Path(in_dir)
        idx = d / "model.safetensors.index.json"
        if idx.exists() and HAVE_SAFETENSORS:
            index = json.loads(idx.read_text())
            files = sorted(set(index["weight_map"].values()))
            hashes = index.get("metadata", {}).get("sha256", {})

            def one(name):
                p = d / name
                if not p.exists():
                    raise CheckpointLoadError(f"missing shard {name}", directory=str(d))
                if self.verify and name in hashes and compute_sha256(p) != hashes[name]:
                    raise CheckpointLoadError(f"sha256 mismatch for {name}", directory=str(d))
                return _st_load(str(p))

            out: dict[str, torch.Tensor] = {}
            with ThreadPoolExecutor(max_workers=self.num_threads) as ex:
                for part in ex.map(one, files):
                    out.update(part)
            return out
        if (d / "model.safetensors").exists() and HAVE_SAFETENSORS:
            return _st_load(str(d / "model.safetensors"))
        for name in ("model.pt", "pytorch_model.bin"):
            if (d / name).exists():
                return torch.load(d / name, map_location="cpu", weights_only=True)
        raise CheckpointLoadError(f"no model weights found in {d}")


def load_pretrained(path: str | os.PathLike, dtype=torch.bfloat16, device=None):
    """Build the framework decoder from a local HF-format directory (config.json + safetensors)."""
    from ..models.llama import LlamaConfig, build_model
    p = Path(path)
    cfg = LlamaConfig.from_dict(json.loads((p / "config.json").read_text()))
    model = build_model(cfg, dtype=dtype, device=device)
    model.load_hf_state_dict(ModelDeserializer().load(p), strict=True)
    return model


def generate_model_card(model_name, base_model: str = "", config: dict | None = None, metrics: dict | None = None,
                        tags: list[str] | None = None, *, model=None, description: str = "",
                        training_config: dict | None = None, serialization_info=None, license: str = "",   # noqa: A002
                        language: str | list | None = None) -> str:
    """README.md text with the YAML front matter the hub reads.  The reference's calling form
    `generate_model_card(model, model_name, description=..., training_config=..., serialization_info=...)` is taken as
    well: a module as first argument supplies the parameter count, `training_config` is `config`."""
    if not isinstance(model_name, str):              # (model, model_name, ...): shift
        model, model_name, base_model = model_name, base_model, ""
    config = config if config is not None else training_config
    tags = tags or ["trainscale-b200"]
    front = ["---", "library_name: trainscale-b200", f"base_model: {base_model}" if base_model else "base_model: none"]
    if license:
        front.append(f"license: {license}")
    if language:
        front += ["language:"] + [f"- {l}" for l in ([language] if isinstance(language, str) else language)]
    lines = front + ["tags:"] + [f"- {t}" for t in tags] + ["---", "", f"# {model_name}", ""]
    if description:
        lines += [description, ""]
    if model is not None and hasattr(model, "parameters"):
        n = sum(p.numel() for p in model.parameters())
        lines += ["## Model", "", f"- **Parameters**: {n:,}", f"- **Class**: {type(model).__name__}", ""]
    if serialization_info is not None:
        lines += ["## Files", "", f"- **Format**: {getattr(serialization_info, 'format', '?')}",
                  f"- **Shards**: {len(getattr(serialization_info, 'shards', ()))}",
                  f"- **Bytes**: {getattr(serialization_info, 'total_bytes', 0):,}", ""]
    if metrics:
        lines += ["## Metrics", ""] + [f"- **{k}**: {v}" for k, v in metrics.items()] + [""]
    if config:
        lines += ["## Training configuration", "", "```json", json.dumps(config, indent=2, default=str), "```", ""]
    return "\n".join(lines)


class HubManager:
    """Thin wrapper over `huggingface_hub` with retry + circuit breaker; a no-op target directory when offline."""

    @reference_kwargs(config="repo_id")
    def __init__(self, repo_id: "str | HubConfig | None" = None, token: str | None = None, private: bool = False,
                 policy: RetryPolicy | None = None):
        self._config = None
        if repo_id is not None and not isinstance(repo_id, str):       # HubManager(HubConfig(...)), the reference's form
            self._config = cfg = repo_id
            repo_id, token, private = cfg.repo_id, token or cfg.token, cfg.private
            policy = policy or RetryPolicy(max_attempts=max(1, cfg.max_retries))
        self.repo_id, self.token, self.private = repo_id, token or os.environ.get("HF_TOKEN"), private
        self.policy, self.breaker = policy or RetryPolicy(), CircuitBreaker()
        self._api = None

    # ---- model-level operations returning Result (data_pipeline/trainer/hub/__init__.py:917-1247)
    @property
    def config(self) -> "HubConfig":
        if self._config is None:
            self._config = HubConfig(repo_id=self.repo_id, token=self.token, private=self.private,
                                     max_retries=self.policy.max_attempts)
        return self._config

    @property
    def api(self):
        """The `huggingface_hub.HfApi` client, created on first use; ImportError when the package is absent."""
        if self._api is None:
            from huggingface_hub import HfApi
            self._api = HfApi(token=self.token)
        return self._api

    def _fail(self, exc: BaseException, **ctx):
        from ..core.types import Err
        return Err(HubError(str(exc), code=classify_hub_error(exc), **ctx))

    def push_to_hub(self, model, repo_id: str | None = None, commit_message: str = "Upload model",
                    model_card: str | None = None, tags: list[str] | None = None, progress_callback=None,
                    local_dir: str | os.PathLike | None = None):
        """Serialise `model` (sharded safetensors + index, config.json when the model has a config, README.md) and
        upload the folder.  `local_dir` keeps the serialised folder; otherwise a temporary one is used.  Ok(url) or
        Err(HubError with a `code` of HubErrorCode)."""
        import tempfile
        from ..core.types import Err, Ok
        repo = repo_id or self.repo_id
        if not repo:
            return Err(HubError("repo_id required for push operation", code=HubErrorCode.VALIDATION_ERROR))
        t0 = time.time_ns()
        tmp = None if local_dir is not None else tempfile.TemporaryDirectory(prefix="ts_hub_")
        out = Path(local_dir if local_dir is not None else tmp.name)
        nbytes = 0
        try:
            res = ModelSerializer(self.config.shard_size_bytes, self.config.prefer_safetensors).serialize(model, out, repo)
            if res.is_err():
                return res
            nbytes = res.unwrap().total_bytes
            cfg = getattr(model, "config", None)
            if cfg is not None:
                d = cfg.to_dict() if hasattr(cfg, "to_dict") else {k: v for k, v in vars(cfg).items()
                                                                   if isinstance(v, (int, float, str, bool, list, type(None)))}
                (out / "config.json").write_text(json.dumps(d, indent=2, default=str))
            (out / "README.md").write_text(model_card or generate_model_card(repo.split("/")[-1], tags=tags))
            if progress_callback is not None:
                progress_callback(0, nbytes)
            old_repo, self.repo_id = self.repo_id, repo
            try:
                if not self.available():
                    raise ImportError("huggingface_hub with a token is needed to upload (offline: the folder is in local_dir)")
                url = self.push(out, commit_message)
            finally:
                self.repo_id = old_repo
            if progress_callback is not None:
                progress_callback(nbytes, nbytes)
            _HUB_METRICS.record_upload(nbytes, time.time_ns() - t0, True)
            return Ok(url)
        except Exception as e:   # noqa: BLE001 - every failure becomes a classified Err
            _HUB_METRICS.record_upload(nbytes, time.time_ns() - t0, False)
            return self._fail(e, repo_id=repo)
        finally:
            if tmp is not None:
                tmp.cleanup()

    def pull_from_hub(self, repo_id: str | None = None, revision: str = "main", cache_dir: str | None = None):
        """Ok(path of the snapshot) or Err.  A `repo_id` that is an existing local directory is returned as it is, so
        that offline hosts can point at a folder written by `push_to_hub(local_dir=...)`."""
        from ..core.types import Err, Ok
        repo = repo_id or self.repo_id
        if not repo:
            return Err(HubError("repo_id required for pull operation", code=HubErrorCode.VALIDATION_ERROR))
        if Path(repo).is_dir():
            return Ok(Path(repo))
        t0 = time.time_ns()
        try:
            from huggingface_hub import snapshot_download
            path = Path(execute_with_retry(lambda: snapshot_download(repo, revision=revision, token=self.token,
                                                                     cache_dir=cache_dir or self.config.cache_dir),
                                           self.policy, self.breaker))
            size = sum(f.stat().st_size for f in path.rglob("*") if f.is_file())
            _HUB_METRICS.record_download(size, time.time_ns() - t0, True)
            return Ok(path)
        except Exception as e:   # noqa: BLE001
            _HUB_METRICS.record_download(0, time.time_ns() - t0, False)
            return self._fail(e, repo_id=repo, revision=revision)

    def load_from_hub(self, model, repo_id: str | None = None, revision: str = "main", strict: bool = True):
        """Weights of the repository (or local folder) loaded into `model`: Ok(model) or Err."""
        from ..core.types import Ok
        got = self.pull_from_hub(repo_id, revision)
        if got.is_err():
            return got
        try:
            sd = ModelDeserializer(self.config.verify_integrity, self.config.max_workers).load(got.unwrap())
            model.load_state_dict(sd, strict=strict)
            return Ok(model)
        except Exception as e:   # noqa: BLE001
            return self._fail(e, strict=strict)

    def get_metrics(self) -> dict:
        return _HUB_METRICS.summary()

    def available(self) -> bool:
        try:
            import huggingface_hub  # noqa: F401
            return bool(self.repo_id and self.token)
        except Exception:
            return False

    def push(self, folder: str | os.PathLike, commit_message: str = "upload") -> str | None:
        if not self.available():
            return None
        from huggingface_hub import HfApi
        api = HfApi(token=self.token)

        def go():
            api.create_repo(self.repo_id, private=self.private, exist_ok=True)
            return api.upload_folder(repo_id=self.repo_id, folder_path=str(folder), commit_message=commit_message)

        return str(execute_with_retry(go, self.policy, self.breaker))

    def pull(self, local_dir: str | os.PathLike) -> str | None:
        if not self.available():
            return None
        from huggingface_hub import snapshot_download
        return execute_with_retry(lambda: snapshot_download(self.repo_id, local_dir=str(local_dir), token=self.token),
                                  self.policy, self.breaker)


class CheckpointManager:
    """Atomic directory checkpoints with metadata, pruning and best / latest tracking."""

    @reference_kwargs(save_dir="root", hub_manager="hub", max_checkpoints="save_total_limit")
    def __init__(self, root: str | os.PathLike, save_total_limit: int = 3, metric: str = "eval_loss",
                 greater_is_better: bool = False, hub: HubManager | None = None):
        self.root, self.limit, self.metric, self.greater, self.hub = Path(root), save_total_limit, metric, greater_is_better, hub
        self.root.mkdir(parents=True, exist_ok=True)
        self.best_value: float | None = None

    def save(self, *args, **kwargs):
        """`save(step, writer, metrics=None)`: `writer(dir)` fills the checkpoint folder; returns its path.
        The reference's form `save(model, optimizer=None, step=0, epoch=0, loss=inf, extra_state=None)` (a module first,
        or `model=`) writes the weights (safetensors), `optimizer.pt` and `training_state.json` itself and returns
        Ok(CheckpointMetadata) / Err(HubError)."""
        ref = bool(args and isinstance(args[0], torch.nn.Module)) or "model" in kwargs
        names = ("model", "optimizer", "step", "epoch", "loss", "extra_state") if ref else ("step", "writer", "metrics")
        if len(args) > len(names):
            raise TypeError(f"save() takes at most {len(names)} positional arguments")
        bound = dict(zip(names, args))
        for k, v in kwargs.items():
            if k in bound:
                raise TypeError(f"save() got multiple values for argument {k!r}")
            if k not in names:
                raise TypeError(f"save() got an unexpected keyword argument {k!r}")
            bound[k] = v
        if ref:
            return self._save_model(bound["model"], bound.get("optimizer"), int(bound.get("step", 0)),
                                    int(bound.get("epoch", 0)), float(bound.get("loss", float("inf"))),
                                    bound.get("extra_state"))
        return self._save_with(int(bound["step"]), bound["writer"], bound.get("metrics"))

    def _save_model(self, model, optimizer, step: int, epoch: int, loss: float, extra_state: dict | None):
        from ..core.types import Err, Ok
        state = {"step": step, "epoch": epoch, "loss": loss, **(extra_state or {})}

        def write(d: Path):
            r = ModelSerializer().serialize(model, d, f"checkpoint-{step}")
            if r.is_err():
                raise r.error
            if optimizer is not None:
                torch.save(optimizer.state_dict(), d / "optimizer.pt")
            (d / "training_state.json").write_text(json.dumps(state, indent=2, default=str))
        try:
            path = self._save_with(step, write, {"epoch": epoch, "loss": loss, self.metric: loss})
            return Ok(CheckpointMetadata.read(path))
        except Exception as e:   # noqa: BLE001
            return Err(HubError(f"failed to save checkpoint: {e}", code=HubErrorCode.SERIALIZATION_ERROR))

    def _save_with(self, step: int, writer: Callable[[Path], None], metrics: dict | None = None) -> Path:
        final = self.root / f"checkpoint-{step}"
        tmp = self.root / f".tmp-checkpoint-{step}"
        if tmp.exists():
            shutil.rmtree(tmp)
        tmp.mkdir(parents=True)
        writer(tmp)
        (tmp / "checkpoint_meta.json").write_text(json.dumps({"step": step, "metrics": metrics or {}, "time": time.time()}))
        if final.exists():
            shutil.rmtree(final)
        os.replace(tmp, final)
        (self.root / "latest").write_text(final.name)
        v = (metrics or {}).get(self.metric)
        if v is not None and (self.best_value is None or (v > self.best_value if self.greater else v < self.best_value)):
            self.best_value = v
            (self.root / "best").write_text(final.name)
        self._prune_old_checkpoints()
        if self.hub is not None:
            self.hub.push(final, f"checkpoint {step}")
        return final

    def list(self) -> list[Path]:
        out = [(int(p.name.split("-")[1]), p) for p in self.root.glob("checkpoint-*") if p.name.split("-")[1].isdigit()]
        return [p for _, p in sorted(out)]

    def latest(self) -> Path | None:
        f = self.root / "latest"
        if f.exists() and (self.root / f.read_text().strip()).exists():
            return self.root / f.read_text().strip()
        all_ = self.list()
        return all_[-1] if all_ else None

    def best(self) -> Path | None:
        f = self.root / "best"
        return self.root / f.read_text().strip() if f.exists() else None

    def get_latest_checkpoint(self) -> "CheckpointMetadata | None":
        p = self.latest()
        return CheckpointMetadata.read(p) if p is not None and (p / "checkpoint_meta.json").exists() else None

    def get_best_checkpoint(self) -> "CheckpointMetadata | None":
        """The checkpoint `best` points at (best value of the tracked metric), else the one with the lowest loss."""
        p = self.best()
        if p is not None and (p / "checkpoint_meta.json").exists():
            return CheckpointMetadata.read(p)
        metas = [CheckpointMetadata.read(d) for d in self.list() if (d / "checkpoint_meta.json").exists()]
        metas = [m for m in metas if m.loss == m.loss]          # drop NaN (no loss recorded)
        return min(metas, key=lambda m: m.loss) if metas else None

    def _prune_old_checkpoints(self):
        if not self.limit or self.limit <= 0:
            return
        keep = {p.name for p in self.list()[-self.limit:]}
        b = self.best()
        if b is not None:
            keep.add(b.name)
        for p in self.list():
            if p.name not in keep:
                shutil.rmtree(p, ignore_errors=True)


# ------------------------------------------------------------------------------------------------ reference surface
import threading as _threading  # noqa: E402
from datetime import datetime as _datetime  # noqa: E402
from enum import Enum as _Enum  # noqa: E402


class HubErrorCode(_Enum):
    """Failure modes of a hub operation (data_pipeline/trainer/hub/__init__.py:80); `classify_hub_error` maps an
    exception onto one, and `RETRIABLE` says which are worth another attempt."""
    NETWORK_FAILURE = "network_failure"
    AUTHENTICATION_FAILED = "authentication_failed"
    REPOSITORY_NOT_FOUND = "repository_not_found"
    PERMISSION_DENIED = "permission_denied"
    QUOTA_EXCEEDED = "quota_exceeded"
    VALIDATION_ERROR = "validation_error"
    SERIALIZATION_ERROR = "serialization_error"
    INTEGRITY_CHECK_FAILED = "integrity_check_failed"
    CIRCUIT_OPEN = "circuit_open"
    DEPENDENCY_MISSING = "dependency_missing"
    TIMEOUT = "timeout"
    RESOURCE_EXHAUSTED = "resource_exhausted"
    INTERNAL_ERROR = "internal_error"


RETRIABLE = frozenset({HubErrorCode.NETWORK_FAILURE, HubErrorCode.TIMEOUT})


def classify_hub_error(exc: BaseException) -> HubErrorCode:
    status = getattr(getattr(exc, "response", None), "status_code", None)
    by_status = {401: HubErrorCode.AUTHENTICATION_FAILED, 403: HubErrorCode.PERMISSION_DENIED,
                 404: HubErrorCode.REPOSITORY_NOT_FOUND, 413: HubErrorCode.QUOTA_EXCEEDED,
                 429: HubErrorCode.QUOTA_EXCEEDED}
    if status in by_status:
        return by_status[status]
    if isinstance(exc, TimeoutError):
        return HubErrorCode.TIMEOUT
    if isinstance(exc, (ImportError, ModuleNotFoundError)):
        return HubErrorCode.DEPENDENCY_MISSING
    if isinstance(exc, MemoryError) or (isinstance(exc, OSError) and getattr(exc, "errno", None) == 28):
        return HubErrorCode.RESOURCE_EXHAUSTED
    if isinstance(exc, (ConnectionError, OSError)):
        return HubErrorCode.NETWORK_FAILURE
    if isinstance(exc, (ValueError, TypeError)):
        return HubErrorCode.VALIDATION_ERROR
    return HubErrorCode.INTERNAL_ERROR


class CircuitState(_Enum):
    CLOSED = "closed"
    OPEN = "open"
    HALF_OPEN = "half_open"

    @classmethod
    def of(cls, breaker: CircuitBreaker) -> "CircuitState":
        breaker.allow()                      # lets an expired open state move to half-open
        return cls(breaker.state)


@dataclass
class HubConfig:
    """Options of hub traffic; the token falls back to HF_TOKEN / HUGGING_FACE_HUB_TOKEN."""
    shard_size_bytes: int = 5 * 2 ** 30
    upload_timeout_s: float = 3600.0
    download_timeout_s: float = 3600.0
    repo_id: str | None = None
    token: str | None = None
    cache_dir: str | None = None
    max_workers: int = 4
    max_retries: int = 3
    private: bool = False
    verify_integrity: bool = True
    prefer_safetensors: bool = True

    def __post_init__(self):
        if self.token is None:
            self.token = os.environ.get("HF_TOKEN") or os.environ.get("HUGGING_FACE_HUB_TOKEN")
        if self.shard_size_bytes <= 0 or self.max_retries < 0:
            raise ValueError("shard_size_bytes must be positive and max_retries non-negative")

    def manager(self) -> HubManager:
        return HubManager(self.repo_id, self.token, self.private, RetryPolicy(max_attempts=max(1, self.max_retries)))

    def serializer(self) -> ModelSerializer:
        return ModelSerializer(self.shard_size_bytes)


class HubMetrics:
    """Counters and latency samples of uploads / downloads, safe to update from several threads."""

    def __init__(self):
        self._lock = _threading.Lock()
        self.uploads_total = self.uploads_failed = self.downloads_total = self.downloads_failed = 0
        self.bytes_uploaded = self.bytes_downloaded = self.retries_total = 0
        self._up_ns: list[int] = []
        self._down_ns: list[int] = []

    def record_upload(self, bytes_count: int, latency_ns: int, success: bool) -> None:
        with self._lock:
            self.uploads_total += 1
            self.uploads_failed += not success
            self.bytes_uploaded += bytes_count if success else 0
            self._up_ns.append(latency_ns)

    def record_download(self, bytes_count: int, latency_ns: int, success: bool) -> None:
        with self._lock:
            self.downloads_total += 1
            self.downloads_failed += not success
            self.bytes_downloaded += bytes_count if success else 0
            self._down_ns.append(latency_ns)

    def record_retry(self) -> None:
        with self._lock:
            self.retries_total += 1

    @staticmethod
    def _pct(xs: list[int], q: float) -> float:
        if not xs:
            return 0.0
        s = sorted(xs)
        return s[min(len(s) - 1, int(q * len(s)))] / 1e6

    def get_percentile_latency_ns(self, percentile: float, operation: str = "upload") -> int | None:
        """`percentile` in [0, 100]; None before the first sample."""
        with self._lock:
            xs = sorted(self._up_ns if operation == "upload" else self._down_ns)
        return xs[min(len(xs) - 1, int(len(xs) * percentile / 100.0))] if xs else None

    def snapshot(self) -> dict:
        """Nested form of `summary()` (data_pipeline/trainer/hub/__init__.py:241-262)."""
        ms = lambda p, op: (self.get_percentile_latency_ns(p, op) or 0) / 1e6      # noqa: E731
        return {"uploads": {"total": self.uploads_total, "failed": self.uploads_failed, "bytes": self.bytes_uploaded,
                            "p50_latency_ms": ms(50, "upload"), "p99_latency_ms": ms(99, "upload")},
                "downloads": {"total": self.downloads_total, "failed": self.downloads_failed,
                              "bytes": self.bytes_downloaded, "p50_latency_ms": ms(50, "download"),
                              "p99_latency_ms": ms(99, "download")},
                "retries_total": self.retries_total}

    def summary(self) -> dict:
        with self._lock:
            return {"uploads_total": self.uploads_total, "uploads_failed": self.uploads_failed,
                    "downloads_total": self.downloads_total, "downloads_failed": self.downloads_failed,
                    "bytes_uploaded": self.bytes_uploaded, "bytes_downloaded": self.bytes_downloaded,
                    "retries_total": self.retries_total, "upload_p50_ms": self._pct(self._up_ns, 0.5),
                    "upload_p99_ms": self._pct(self._up_ns, 0.99), "download_p50_ms": self._pct(self._down_ns, 0.5)}


_HUB_METRICS = HubMetrics()


def get_hub_metrics() -> HubMetrics:
    return _HUB_METRICS


@dataclass(frozen=True)
class ShardInfo:
    filename: str
    byte_offset: int
    byte_size: int
    sha256: str
    tensor_names: tuple


@dataclass(frozen=True)
class SerializationResult:
    shards: tuple
    total_bytes: int
    format: str
    metadata: dict

    @classmethod
    def describe(cls, out_dir: str | os.PathLike) -> "SerializationResult":
        """What `ModelSerializer.save` left in `out_dir`, from the index (or the single file)."""
        out = Path(out_dir)
        idx = out / "model.safetensors.index.json"
        if idx.exists():
            index = json.loads(idx.read_text())
            by_file: dict[str, list[str]] = {}
            for k, f in index["weight_map"].items():
                by_file.setdefault(f, []).append(k)
            hashes = index.get("metadata", {}).get("sha256", {})
        else:
            single = [p.name for p in (out / "model.safetensors", out / "model.pt") if p.exists()]
            by_file, hashes = {f: [] for f in single}, {}
        shards, off = [], 0
        for f in sorted(by_file):
            size = (out / f).stat().st_size
            shards.append(ShardInfo(f, off, size, hashes.get(f) or compute_sha256(out / f), tuple(by_file[f])))
            off += size
        fmt = "safetensors" if any(s.filename.endswith(".safetensors") for s in shards) else "pytorch"
        return cls(tuple(shards), off, fmt, {"num_shards": len(shards)})


@dataclass(frozen=True)
class CheckpointMetadata:
    step: int
    epoch: int
    loss: float
    timestamp: _datetime
    sha256: str
    path: Path

    @classmethod
    def read(cls, checkpoint_dir: str | os.PathLike) -> "CheckpointMetadata":
        """From the `checkpoint_meta.json` a `CheckpointManager` writes; the hash covers that file."""
        d = Path(checkpoint_dir)
        meta = json.loads((d / "checkpoint_meta.json").read_text())
        m = meta.get("metrics", {})
        return cls(int(meta.get("step", 0)), int(m.get("epoch", 0)), float(m.get("loss", m.get("eval_loss", float("nan")))),
                   _datetime.fromtimestamp(meta.get("time", 0.0)), compute_sha256(d / "checkpoint_meta.json"), d)


# ---- defaults of data_pipeline/trainer/hub/__init__.py, as the classes above use them
CACHE_LINE_SIZE = 64
DEFAULT_SHARD_SIZE_BYTES = 5 * 1024 ** 3
MAX_RETRY_ATTEMPTS, INITIAL_BACKOFF_MS, MAX_BACKOFF_MS = 5, 100, 32000
IO_BUFFER_SIZE, HASH_CHUNK_SIZE = 8 * 1024 * 1024, 1024 * 1024
CIRCUIT_BREAKER_THRESHOLD, CIRCUIT_BREAKER_TIMEOUT_S = 3, 60.0
UPLOAD_CONCURRENCY = min(8, (os.cpu_count() or 4) + 4)
