"""Throughput / MFU accounting on device timers.

tokens/s is computed from CUDA-event durations (never host wall-clock of one micro-step, which is what
data_pipeline/trainer/trainers/sota_trainer.py:2389-2398 does); MFU = achieved FLOP/s over a peak.  Peak table as
in data_pipeline/trainer/metrics/throughput.py:30-47 with B200 dense bf16 = 2250 TFLOPS; a measured peak (e.g.
from MEASURED_PEAKS.json) can be passed instead.
"""
from __future__ import annotations

import json
import time
from collections import deque
from pathlib import Path

import torch
from ..utils.refargs import ANY, reference_kwargs  # noqa: F401

PEAK_TFLOPS = {"B200": 2250.0, "H200": 989.0, "H100": 989.0, "A100": 312.0, "L40S": 362.0, "A10": 125.0, "T4": 65.0,
               "V100": 125.0, "RTX 4090": 330.0, "RTX 3090": 142.0}


def device_peak_tflops(device=None, measured_file: str | None = None) -> float:
    if measured_file and Path(measured_file).exists():
        try:
            return float(json.loads(Path(measured_file).read_text())["bf16_tflops"])
        except Exception:
            pass
    if torch.cuda.is_available():
        name = torch.cuda.get_device_name(device)
        for k, v in PEAK_TFLOPS.items():
            if k in name:
                return v
    return 1.0


class ThroughputTracker:
    def __init__(self, flops_per_token: float = 0.0, peak_tflops: float | None = None, window: int = 20,
                 world_size: int = 1, use_cuda_events: bool | None = None):
        self.flops_per_token, self.world_size = flops_per_token, world_size
        self.peak = peak_tflops if peak_tflops is not None else device_peak_tflops()
        self.cuda = torch.cuda.is_available() if use_cuda_events is None else use_cuda_events
        self.window = deque(maxlen=window)
        self.total_tokens = 0
        self.total_seconds = 0.0
        self.total_samples = 0
        self.step_count = 0
        self._pending: list[tuple] = []
        self._t0 = None
        self._started = self._last = None

    def start_step(self):
        if self.cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            self._t0 = time.perf_counter()

    def end_step(self, tokens_this_rank: int):
        if self._t0 is None:
            return
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pending.append((self._t0, e, tokens_this_rank))
        else:
            self._add(time.perf_counter() - self._t0, tokens_this_rank)
        self._t0 = None

    def _add(self, seconds, tokens):
        tokens *= self.world_size
        self.window.append((seconds, tokens))
        self.total_tokens += tokens
        self.total_seconds += seconds

    def flush(self):
        """Read finished events (non-blocking for events that are not complete yet)."""
        keep = []
        for a, b, n in self._pending:
            if b.query():
                self._add(a.elapsed_time(b) / 1e3, n)
            else:
                keep.append((a, b, n))
        self._pending = keep

    def tokens_per_second(self) -> float:
        self.flush()
        s = sum(x for x, _ in self.window)
        return sum(t for _, t in self.window) / s if s > 0 else 0.0

    def tflops(self) -> float:
        return self.tokens_per_second() * self.flops_per_token / 1e12

    def compute_mfu(self, model_params: int | None = None, peak_tflops: float | None = None, *,
                    flops_per_token: float | None = None, seq_len: int | None = None) -> float:
        """Achieved FLOP/s over the peak of all GPUs.  FLOPs per token: `flops_per_token` when given, else the tracker's
        own figure, or 6 x `model_params` (forward + backward of a dense decoder, attention not counted) when that is
        given.  `seq_len` is accepted for the reference's signature; the 6 N estimate does not depend on it."""
        denom = (peak_tflops if peak_tflops is not None else self.peak) * self.world_size
        if flops_per_token is not None:
            rate = self.tokens_per_second() or self.tokens_per_sec()
            return rate * float(flops_per_token) / 1e12 / denom if denom > 0 else 0.0
        if model_params:
            rate = self.tokens_per_second() or self.tokens_per_sec()
            return rate * 6.0 * model_params / 1e12 / denom if denom > 0 else 0.0
        return self.tflops() / denom if denom > 0 else 0.0

    def state_dict(self):
        return {"total_tokens": self.total_tokens, "total_seconds": self.total_seconds,
                "total_samples": self.total_samples, "step_count": self.step_count}

    @reference_kwargs(state="sd")
    def load_state_dict(self, sd):
        self.total_tokens, self.total_seconds = sd["total_tokens"], sd["total_seconds"]
        self.total_samples, self.step_count = sd.get("total_samples", 0), sd.get("step_count", 0)

    # ---- wall-clock interface of the reference (data_pipeline/trainer/metrics/throughput.py:137-360): `start()`,
    # then `update(samples, tokens)` once per step; rates are totals over the time since `start()`, or over the last
    # `window` steps.  The CUDA-event interface above (`start_step` / `end_step`) feeds the same totals.
    def reset(self) -> None:
        self.window.clear()
        self.total_tokens, self.total_seconds, self.total_samples, self.step_count = 0, 0.0, 0, 0
        self._pending, self._t0, self._started, self._last = [], None, None, None

    def start(self) -> None:
        self._started = self._last = time.perf_counter()

    def update(self, samples: int = 0, tokens: int = 0, flops: float = 0.0) -> None:
        now = time.perf_counter()
        if self._started is None:
            self.start()
            now = self._started
        dt = now - self._last
        self._last = now
        self.total_samples += samples * self.world_size
        self.step_count += 1
        if dt > 0:
            self._add(dt, tokens)
        else:
            self.total_tokens += tokens * self.world_size

    def elapsed_seconds(self) -> float:
        return (time.perf_counter() - self._started) if self._started is not None else self.total_seconds

    def samples_per_sec(self) -> float:
        s = self.elapsed_seconds()
        return self.total_samples / s if s > 0 else 0.0

    def tokens_per_sec(self) -> float:
        self.flush()
        s = self.elapsed_seconds() if self._started is not None else self.total_seconds
        return self.total_tokens / s if s > 0 else 0.0

    def tokens_per_sec_window(self) -> float:
        return self.tokens_per_second()

    def compute_tflops(self, flops_per_token: float | None = None) -> float:
        f = self.flops_per_token if flops_per_token is None else flops_per_token
        return self.tokens_per_sec() * f / 1e12

    def sync(self, process_group=None) -> None:
        """No-op when totals already count all ranks (`world_size` > 1 at construction); otherwise sum them."""
        import torch.distributed as dist
        if self.world_size > 1 or not (dist.is_available() and dist.is_initialized()):
            return
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(process_group) == "nccl" else "cpu"
        t = torch.tensor([float(self.total_tokens), float(self.total_samples)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, group=process_group)
        self.total_tokens, self.total_samples = int(t[0]), int(t[1])

    def log_dict(self) -> dict:
        return {"throughput/tokens_per_sec": self.tokens_per_sec(), "throughput/samples_per_sec": self.samples_per_sec(),
                "throughput/tokens_per_sec_window": self.tokens_per_sec_window(), "throughput/mfu": self.compute_mfu(),
                "throughput/total_tokens": float(self.total_tokens), "throughput/elapsed_seconds": self.elapsed_seconds()}
