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
        self._pending: list[tuple] = []
        self._t0 = None

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

    def compute_mfu(self) -> float:
        denom = self.peak * self.world_size
        return self.tflops() / denom if denom > 0 else 0.0

    def state_dict(self):
        return {"total_tokens": self.total_tokens, "total_seconds": self.total_seconds}

    def load_state_dict(self, sd):
        self.total_tokens, self.total_seconds = sd["total_tokens"], sd["total_seconds"]
