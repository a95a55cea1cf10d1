"""Phase markers and optional traces.

* `nvtx_range(name)`: NVTX range around a phase (forward / backward / optimizer / a collective) so that a timeline
  tool groups the framework's kernels by phase.  Off unless TS_NVTX=1 (or `enable_nvtx(True)`): the ranges cost a
  host call each and the hot loop makes none by default.
* `profile_steps(...)`: a `torch.profiler` schedule (wait / warm-up / active) that writes a chrome trace (and
  TensorBoard files when a handler directory is given), stepped once per optimizer step.
* `PhaseTimer`: CUDA-event timing of named phases, read after the fact (no host sync in the step).

The reference has `record_function` + a profiler context only in its pipeline module
(data_pipeline/trainer/distributed/pipeline_parallel.py:2293, 2580-2619) and no NVTX ranges.
"""
from __future__ import annotations

import contextlib
import os
from pathlib import Path

import torch

_NVTX = {"on": os.environ.get("TS_NVTX", "0") == "1"}


def enable_nvtx(on: bool = True) -> None:
    _NVTX["on"] = bool(on)


def nvtx_enabled() -> bool:
    return _NVTX["on"] and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    if not nvtx_enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_mark(name: str) -> None:
    if nvtx_enabled():
        torch.cuda.nvtx.mark(name)


class PhaseTimer:
    """`with timer("forward"): ...` records an event pair per use; `summary()` reads the pairs that have completed.
    On CPU it falls back to a wall clock."""

    def __init__(self, device: torch.device | str | None = None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._pending: list[tuple[str, object, object]] = []
        self._ms: dict[str, float] = {}
        self._n: dict[str, int] = {}

    @contextlib.contextmanager
    def __call__(self, name: str):
        with nvtx_range(name):
            if self.cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                try:
                    yield
                finally:
                    b.record()
                    self._pending.append((name, a, b))
            else:
                import time
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._add(name, (time.perf_counter() - t0) * 1e3)

    def _add(self, name: str, ms: float) -> None:
        self._ms[name] = self._ms.get(name, 0.0) + ms
        self._n[name] = self._n.get(name, 0) + 1

    def flush(self) -> None:
        keep = []
        for name, a, b in self._pending:
            if b.query():
                self._add(name, a.elapsed_time(b))
            else:
                keep.append((name, a, b))
        self._pending = keep

    def summary(self) -> dict[str, dict[str, float]]:
        self.flush()
        return {k: {"total_ms": v, "count": self._n[k], "mean_ms": v / self._n[k]} for k, v in self._ms.items()}


@contextlib.contextmanager
def profile_steps(out_dir: str | os.PathLike, wait: int = 1, warmup: int = 1, active: int = 3, tensorboard: bool = False,
                  record_shapes: bool = False, with_stack: bool = False):
    """Yields an object with `.step()`; call it once per optimizer step.  After wait + warm-up, `active` steps are
    traced and written to `<out_dir>/trace_<n>.json` (chrome://tracing / Perfetto)."""
    from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    count = {"n": 0}

    def on_ready(prof):
        if tensorboard:
            tensorboard_trace_handler(str(out))(prof)
        else:
            prof.export_chrome_trace(str(out / f"trace_{count['n']}.json"))
        count["n"] += 1

    with profile(activities=acts, schedule=schedule(wait=wait, warmup=warmup, active=active, repeat=1),
                 on_trace_ready=on_ready, record_shapes=record_shapes, with_stack=with_stack) as prof:
        yield prof
