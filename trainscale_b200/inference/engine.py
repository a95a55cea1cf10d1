"""Inference engine: paged KV cache, continuous batching with chunked prefill, sampling, streaming, an
OpenAI-compatible HTTP server and a CLI.

API surface after data_pipeline/trainer/inference.py:229-2421 (`EngineConfig` with scheduler / cache / parallel /
speculative / LoRA / observability sub-configs, `GenerationParams`, `RequestMetrics` with TTFT / TPOT, percentile
`MetricsAggregator`, `EngineBuilder`, `SOTAInferenceEngine.generate`, `SOTAAsyncStreamEngine.generate_stream /
abort_request`, `EnginePresets`, `create_openai_server` with /v1/completions, /v1/chat/completions, /health,
/metrics, CLI sub-commands probe | batch | stream | serve | bench).  The reference wraps vLLM; this engine runs
the framework's own decoder on its own kernels: flash attention with packed prompts (cu_seqlens) for prefill,
paged split-KV decode attention, tcgen05 GEMMs, fused norms.
"""
from __future__ import annotations

import argparse
import asyncio
import ctypes
import json
import math
import sys
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Any, AsyncIterator, Iterable

import torch

from ..utils.refargs import ANY, reference_kwargs

from ..core.types import Err, Ok, Result
from ..ops import _lib, activation, attention, gemm, norm, rope
from .kv_cache import PagedKVCache
from .sampling import apply_penalties, sample


# ------------------------------------------------------------------------------------------------ configuration
@dataclass
class QuantizationConfig:
    method: str | None = None          # None | fp8 (weights kept bf16 when None)
    kv_cache_dtype: str = "auto"


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 8192
    enable_chunked_prefill: bool = True
    policy: str = "fcfs"


@dataclass
class CacheConfig:
    block_size: int = 16
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks: int | None = None
    enable_prefix_caching: bool = True
    max_model_len: int = 8192


@dataclass
class SpeculativeConfig:
    enabled: bool = False
    draft_model: str | None = None
    num_speculative_tokens: int = 4


@dataclass
class LoRAServingConfig:
    enabled: bool = False
    max_loras: int = 1
    max_lora_rank: int = 64


@dataclass
class ObservabilityConfig:
    collect_metrics: bool = True
    log_requests: bool = False


@dataclass
class EngineConfig:
    model: str = "tiny"                       # preset name or local HF-format directory
    tokenizer: str | None = None              # None -> built-in byte tokenizer unless `model` is a directory
    dtype: str = "bfloat16"
    device: str = "auto"
    seed: int = 0
    quantization: QuantizationConfig = field(default_factory=QuantizationConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    speculative: SpeculativeConfig = field(default_factory=SpeculativeConfig)
    lora: LoRAServingConfig = field(default_factory=LoRAServingConfig)
    observability: ObservabilityConfig = field(default_factory=ObservabilityConfig)
    enforce_eager: bool = True


@dataclass
class GenerationParams:
    max_tokens: int = 128
    temperature: float = 0.7
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    stop: list[str] = field(default_factory=list)
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    seed: int | None = None
    logprobs: bool = False
    n: int = 1
    lora_name: str | None = None        # adapter of this request (see EngineCore.load_adapters)

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.n < 1:
            raise ValueError("n must be >= 1")

    def to_sampling_params(self) -> dict:
        """Validated keyword form of the sampling settings, as the sampler of this engine (or an external one with the
        same vocabulary of options, e.g. vllm.SamplingParams(**d)) takes them; unset options are left out."""
        self.validate()
        d = {"max_tokens": self.max_tokens, "temperature": self.temperature, "top_p": self.top_p,
             "top_k": self.top_k if self.top_k > 0 else -1, "min_p": self.min_p,
             "repetition_penalty": self.repetition_penalty, "frequency_penalty": self.frequency_penalty,
             "presence_penalty": self.presence_penalty, "n": self.n, "ignore_eos": self.ignore_eos}
        if self.seed is not None:
            d["seed"] = self.seed
        if self.stop:
            d["stop"] = list(self.stop)
        if self.stop_token_ids:
            d["stop_token_ids"] = list(self.stop_token_ids)
        if self.logprobs:
            d["logprobs"] = 1
        return d


@dataclass
class RequestMetrics:
    request_id: str = ""
    prompt_tokens: int = 0
    completion_tokens: int = 0
    arrival: float = 0.0
    first_token: float | None = None
    finished: float | None = None
    cached_prompt_tokens: int = 0

    @property
    def ttft(self) -> float | None:
        return None if self.first_token is None else self.first_token - self.arrival

    @property
    def tpot(self) -> float | None:
        if self.finished is None or self.first_token is None or self.completion_tokens < 2:
            return None
        return (self.finished - self.first_token) / (self.completion_tokens - 1)

    @property
    def e2e(self) -> float | None:
        return None if self.finished is None else self.finished - self.arrival

    def mark_submitted(self) -> None:
        self.arrival = time.perf_counter()

    def mark_first_token(self) -> None:
        if self.first_token is None:
            self.first_token = time.perf_counter()

    @reference_kwargs(num_generated="completion_tokens")
    def mark_complete(self, completion_tokens: int | None = None, num_prompt: int | None = None) -> None:
        self.finished = time.perf_counter()
        if completion_tokens is not None:
            self.completion_tokens = completion_tokens
        if num_prompt is not None:
            self.prompt_tokens = num_prompt


class MetricsAggregator:
    def __init__(self):
        self.records: list[RequestMetrics] = []

    def add(self, m: RequestMetrics) -> None:
        self.records.append(m)

    def record(self, metrics: RequestMetrics) -> None:
        self.records.append(metrics)

    def summarize(self) -> dict:
        """`summary()`, or {"status": "no_requests_completed"} before the first finished request."""
        return self.summary() if self.records else {"status": "no_requests_completed"}

    @staticmethod
    def _pct(vals: list[float], p: float) -> float | None:
        if not vals:
            return None
        vals = sorted(vals)
        k = (len(vals) - 1) * p
        lo, hi = math.floor(k), math.ceil(k)
        return vals[lo] + (vals[hi] - vals[lo]) * (k - lo)

    def summary(self) -> dict:
        out = {"requests": len(self.records), "prompt_tokens": sum(r.prompt_tokens for r in self.records),
               "completion_tokens": sum(r.completion_tokens for r in self.records)}
        for name in ("ttft", "tpot", "e2e"):
            vals = [getattr(r, name) for r in self.records if getattr(r, name) is not None]
            for p in (0.5, 0.95, 0.99):
                out[f"{name}_p{int(p * 100)}"] = self._pct(vals, p)
        return out

    def prometheus(self) -> str:
        s = self.summary()
        lines = []
        for k, v in s.items():
            if v is not None:
                lines.append(f"trainscale_inference_{k} {v}")
        return "\n".join(lines) + "\n"


@dataclass
class InferenceResponse:
    request_id: str
    prompt: str
    text: str
    token_ids: list[int]
    finish_reason: str
    metrics: RequestMetrics
    logprobs: list[float] | None = None


@dataclass
class StreamChunk:
    request_id: str
    text: str
    token_id: int
    finished: bool
    finish_reason: str | None = None


# ------------------------------------------------------------------------------------------------ model runner
class ModelRunner:
    """Runs the framework decoder over a flattened token batch with a paged KV cache."""

    def __init__(self, model, cache: PagedKVCache, device, tp=None, use_graphs: bool = False):
        """`tp`: tensor-parallel context of a model sharded with `shard_model_for_tensor_parallel` (every rank runs
        the same batch; the attention and MLP outputs are all-reduced).  `use_graphs`: pure decode steps replay a CUDA
        graph per (padded batch size, block-table width) instead of launching ~12 kernels per layer from Python."""
        self.model, self.cache, self.device = model.eval(), cache, torch.device(device)
        self.cfg = model.config
        self.cuda = self.device.type == "cuda" and next(model.parameters()).dtype == torch.bfloat16
        self.cos, self.sin = model.model.rope_tables(self.device, min(self.cfg.max_position_embeddings, 1 << 16))
        self.lora = None                 # multi_lora.BatchedLoRA when adapters are loaded
        self.tp = tp if (tp is not None and tp.active) else None
        ws = self.tp.size if self.tp is not None else 1
        self.Hq, self.Hkv = self.cfg.num_attention_heads // ws, self.cfg.num_key_value_heads // ws
        self.use_graphs = bool(use_graphs) and self.cuda
        self.graphs: dict = {}
        self.graph_replays = 0

    def _reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None:
            torch.distributed.all_reduce(x, group=self.tp.group)
        return x

    def _lin(self, li: int, wname: str, w: torch.Tensor, x: torch.Tensor, adapter_ids) -> torch.Tensor:
        y = gemm.linear(x, w)
        if self.lora is not None and adapter_ids is not None:
            d = self.lora.delta(li, wname, x, adapter_ids)
            if d is not None:
                y = y + d
        return y

    def _write_cache(self, layer: int, qkv2d: torch.Tensor, slots: torch.Tensor) -> None:
        c = self.cfg
        Hq, Hkv, D = self.Hq, self.Hkv, c.head_dim
        kw = Hkv * D
        if self.cuda:
            lib = _lib.load("decode")
            rc = lib.ts_kv_cache_write(_lib.ptr(qkv2d), qkv2d.stride(0), Hq * D, Hq * D + kw, _lib.ptr(self.cache.k[layer]),
                                       _lib.ptr(self.cache.v[layer]), _lib.ptr(slots), ctypes.c_longlong(qkv2d.shape[0]),
                                       kw, _lib.stream_ptr())
            _lib.check(rc, "ts_kv_cache_write")
        else:
            k = qkv2d[:, Hq * D:Hq * D + kw].view(-1, Hkv, D)
            v = qkv2d[:, Hq * D + kw:].view(-1, Hkv, D)
            self.cache.k[layer].view(-1, Hkv, D)[slots] = k
            self.cache.v[layer].view(-1, Hkv, D)[slots] = v

    def _gathered_kv(self, layer: int, seq_id: int):
        s = self.cache.seqs[seq_id]
        idx = torch.tensor(s.blocks, device=self.device)
        c = self.cfg
        k = self.cache.k[layer][idx].reshape(-1, self.Hkv, c.head_dim)[:s.num_tokens]
        v = self.cache.v[layer][idx].reshape(-1, self.Hkv, c.head_dim)[:s.num_tokens]
        return k, v

    def _attend(self, layer: int, qkv2d: torch.Tensor, seq_ids: list[int], q_lens: list[int], fresh: bool,
                block_table, seq_lens, splits: int | None = None) -> torch.Tensor:
        c = self.cfg
        Hq, Hkv, D = self.Hq, self.Hkv, c.head_dim
        scale = 1.0 / math.sqrt(D)
        T = qkv2d.shape[0]
        if self.cuda and fresh and D in (64, 128):
            # every sequence starts at position 0: packed-prompt flash attention
            from ..ops import flash
            cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0).tolist()), dtype=torch.int32, device=self.device)
            o, _ = flash.flash_forward_only(qkv2d.unsqueeze(0), Hq, Hkv, D, True, scale, cu, max(q_lens))
            return o.view(T, Hq * D)
        if self.cuda and all(n == 1 for n in q_lens) and D in (64, 128):
            lib = _lib.load("decode")
            n = qkv2d.shape[0]
            chunk = 512
            if splits is None:       # (a captured decode passes the split count of its block-table width)
                splits = max(1, -(-int(seq_lens.max().item()) // chunk))
            out = torch.empty(n, Hq * D, dtype=qkv2d.dtype, device=self.device)
            po = torch.empty(n, Hq, splits, D, dtype=torch.float32, device=self.device)
            pl = torch.empty(n, Hq, splits, dtype=torch.float32, device=self.device)
            rc = lib.ts_decode_attention(_lib.ptr(qkv2d), qkv2d.stride(0), _lib.ptr(self.cache.k[layer]),
                                         _lib.ptr(self.cache.v[layer]), _lib.ptr(block_table), block_table.shape[1],
                                         _lib.ptr(seq_lens), _lib.ptr(out), Hq * D, _lib.ptr(po), _lib.ptr(pl), n, Hq,
                                         Hkv, D, self.cache.block_size, chunk, splits, ctypes.c_float(scale),
                                         _lib.stream_ptr())
            _lib.check(rc, "ts_decode_attention")
            return out
        # general path (chunked prefill continuation, CPU): per sequence against the gathered cache
        outs, off = [], 0
        for sid, n in zip(seq_ids, q_lens):
            q = qkv2d[off:off + n, :Hq * D].view(1, n, Hq, D)
            k, v = self._gathered_kv(layer, sid)
            o = attention.attention_reference(q, k.unsqueeze(0), v.unsqueeze(0), True, scale)
            outs.append(o.reshape(n, Hq * D))
            off += n
        return torch.cat(outs)

    def _layers(self, token_ids, pos32, slots, seq_ids, q_lens, fresh, adapter_ids, block_table, seq_lens,
                splits: int | None = None) -> torch.Tensor:
        """The decoder over a flattened token batch; returns the final-norm hidden state of every token."""
        m, c = self.model.model, self.cfg
        x = m.embed_tokens(token_ids)
        if getattr(c, "scale_embeddings", False):
            x = x * torch.tensor(c.hidden_size ** 0.5, dtype=x.dtype)
        res = None
        for li, layer in enumerate(m.layers):
            attn, mlp = getattr(layer.self_attn, "inner", layer.self_attn), getattr(layer.mlp, "inner", layer.mlp)
            h, res = layer.input_layernorm(x, res)
            qkv = self._lin(li, "wqkv", attn.wqkv, h, adapter_ids)
            if attn.bqkv is not None:
                qkv = qkv + attn.bqkv
            qkv = rope.apply_rope_qkv(qkv.unsqueeze(0), self.Hq + self.Hkv, c.head_dim, self.cos, self.sin,
                                      pos32.unsqueeze(0), qkv.shape[0], 0, c.rope_interleaved)[0]
            self._write_cache(li, qkv, slots)
            a = self._attend(li, qkv, seq_ids, q_lens, fresh, block_table, seq_lens, splits)
            a = self._reduce(self._lin(li, "wo", attn.wo, a, adapter_ids))
            h, res = layer.post_attention_layernorm(a, res)
            if hasattr(mlp, "router"):            # mixture of experts: the block routes by itself
                x = layer.mlp(h)
            else:
                x = self._reduce(self._lin(li, "w_down", mlp.w_down,
                                           activation.glu(self._lin(li, "w_gate_up", mlp.w_gate_up, h, adapter_ids),
                                                          mlp.act), adapter_ids))
        x, _ = m.norm(x, res)
        return x

    @torch.no_grad()
    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, seq_ids: list[int],
                q_lens: list[int], fresh: bool, adapter_ids: torch.Tensor | None = None) -> torch.Tensor:
        """token_ids / positions / slots: [T]; returns the hidden state of each sequence's LAST token [n_seq, H].
        `adapter_ids` [T]: LoRA adapter index of every token (requests with different adapters share the batch)."""
        block_table, seq_lens = self.cache.block_table(seq_ids, self.device)
        x = self._layers(token_ids, positions.to(torch.int32), slots, seq_ids, q_lens, fresh, adapter_ids, block_table,
                         seq_lens)
        last = torch.tensor(q_lens, device=self.device).cumsum(0) - 1
        return x[last]

    # ---------------------------------------------------------------- CUDA-graph decode
    def can_graph(self, q_lens: list[int]) -> bool:
        c = self.cfg
        return (self.use_graphs and self.lora is None and all(n == 1 for n in q_lens) and c.head_dim in (64, 128)
                and getattr(c, "num_local_experts", 0) == 0 and len(q_lens) <= 256)

    @torch.no_grad()
    def decode_graphed(self, toks: list[int], pos: list[int], slots: list[int], seq_ids: list[int]) -> torch.Tensor:
        """One decode step (one new token per sequence) replayed from a CUDA graph; returns fp32 logits [n, V].
        The batch is padded to a power of two with rows that write to / read from the cache's spare block."""
        n = len(seq_ids)
        n_pad = 1
        while n_pad < n:
            n_pad *= 2
        bt, sl = self.cache.block_table(seq_ids, None)
        width = -(-bt.shape[1] // 32) * 32
        key = (n_pad, width)
        st = self.graphs.get(key)
        if st is None:
            st = self.graphs[key] = self._capture(n_pad, width)
        bs, trash = self.cache.block_size, self.cache.trash_block
        h = st["host"]
        h["tok"].zero_()
        h["pos"].zero_()
        h["slots"].fill_(trash * bs)
        h["sl"].fill_(1)
        h["bt"].fill_(trash)
        h["tok"][:n] = torch.tensor(toks)
        h["pos"][:n] = torch.tensor(pos, dtype=torch.int32)
        h["slots"][:n] = torch.tensor(slots)
        h["sl"][:n] = sl
        h["bt"][:n, :bt.shape[1]] = bt
        for k in ("tok", "pos", "slots", "sl", "bt"):
            st[k].copy_(h[k], non_blocking=True)
        st["graph"].replay()
        self.graph_replays += 1
        return st["logits"][:n]

    def _capture(self, n_pad: int, width: int) -> dict:
        dev = self.device
        bs, trash = self.cache.block_size, self.cache.trash_block
        st = {"tok": torch.zeros(n_pad, dtype=torch.long, device=dev),
              "pos": torch.zeros(n_pad, dtype=torch.int32, device=dev),
              "slots": torch.full((n_pad,), trash * bs, dtype=torch.long, device=dev),
              "sl": torch.ones(n_pad, dtype=torch.int32, device=dev),
              "bt": torch.full((n_pad, width), trash, dtype=torch.int32, device=dev)}
        st["host"] = {k: torch.empty_like(v, device="cpu").pin_memory() for k, v in st.items()}
        splits = max(1, -(-(width * bs) // 512))
        ids = list(range(n_pad))

        def body():
            x = self._layers(st["tok"], st["pos"], st["slots"], ids, [1] * n_pad, False, None, st["bt"], st["sl"], splits)
            return self.model.logits(x).float()

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            body()                                  # lazy initialisation (library loads, attribute setup) outside capture
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            st["logits"] = body()
        st["graph"] = g
        return st

    @torch.no_grad()
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.model.logits(hidden).float()


# ------------------------------------------------------------------------------------------------ scheduler / engine core
@dataclass
class _Request:
    request_id: str
    prompt: str
    prompt_ids: list[int]
    params: GenerationParams
    metrics: RequestMetrics
    seq_id: int
    output_ids: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    prefilled: int = 0
    generator: torch.Generator | None = None
    finished: bool = False
    finish_reason: str | None = None
    emitted_text_len: int = 0


class EngineCore:
    """Continuous batching: every step packs the decode tokens of running requests plus as many prompt tokens of
    waiting requests as the token budget allows (chunked prefill)."""

    def __init__(self, config: EngineConfig, model=None, tokenizer=None):
        from ..data.tokenization import TokenizerWrapper, create_tokenizer
        from ..models.llama import PRESETS, build_model
        self.config = config
        self.adapter_states: dict[str, dict[str, torch.Tensor]] = {}   # registry behind `load_adapters`
        dev = config.device
        if dev == "auto":
            dev = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(dev)
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[config.dtype]
        if self.device.type == "cpu":
            dtype = torch.float32
        if model is None:
            if config.model in PRESETS:
                model = build_model(config.model, dtype=dtype, device=self.device, seed=config.seed)
            else:
                from ..hub import load_pretrained
                model = load_pretrained(config.model, dtype=dtype, device=self.device)
        self.model = model.to(self.device)
        # tensor-parallel serving: every rank of the (already initialised) process group runs this engine on the same
        # requests with its slice of every projection; sampling uses the same seeds, so all ranks emit the same tokens
        self.tp = None
        tps = int(config.parallel.tensor_parallel_size or 1)
        if tps > 1:
            import torch.distributed as dist
            from ..parallel import tp as TP
            if not dist.is_initialized() or dist.get_world_size() != tps:
                raise ValueError(f"tensor_parallel_size={tps} needs a torch.distributed job of exactly {tps} ranks "
                                 "(launch the engine under torchrun)")
            if getattr(self.model, "tp", None) is None:
                ctx = TP.TPContext.from_group(dist.group.WORLD, sequence_parallel=False, comm="nccl")
                TP.shard_model_for_tensor_parallel(self.model, ctx)
            self.tp = self.model.tp
        if tokenizer is None:
            tokenizer = create_tokenizer(name_or_path=config.tokenizer or ("byte" if config.model in PRESETS else config.model),
                                         padding=False, truncation=False)
        self.tokenizer = tokenizer if isinstance(tokenizer, TokenizerWrapper) else TokenizerWrapper(tokenizer, padding=False)
        c = self.model.config
        cc = config.cache
        nb = cc.num_gpu_blocks
        if nb is None:
            per_block = 2 * c.num_hidden_layers * cc.block_size * (c.num_key_value_heads // tps) * c.head_dim * \
                (2 if dtype != torch.float32 else 4)
            if self.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(self.device)
                nb = max(64, int(free * cc.gpu_memory_utilization * 0.5) // per_block)
            else:
                nb = 512
            nb = min(nb, max(64, cc.max_model_len * config.scheduler.max_num_seqs // cc.block_size + 64))
        self.cache = PagedKVCache(c.num_hidden_layers, nb, cc.block_size, c.num_key_value_heads // tps, c.head_dim, dtype,
                                  self.device, cc.enable_prefix_caching)
        self.runner = ModelRunner(self.model, self.cache, self.device, tp=self.tp, use_graphs=not config.enforce_eager)
        self.waiting: deque[_Request] = deque()
        self.running: list[_Request] = []
        self.metrics = MetricsAggregator()
        self._next_seq = 0
        self.steps = 0

    # -------------------------------------------------------------- requests
    def add_request(self, prompt: str | list[int], params: GenerationParams | None = None, request_id: str | None = None) -> _Request:
        params = params or GenerationParams()
        params.validate()
        ids = list(prompt) if not isinstance(prompt, str) else self.tokenizer.encode_raw(prompt, add_special_tokens=False)
        if isinstance(prompt, str) and self.tokenizer.bos_token_id is not None:
            ids = [self.tokenizer.bos_token_id] + ids
        if not ids:
            ids = [self.tokenizer.bos_token_id or 0]
        max_len = self.config.cache.max_model_len
        if len(ids) >= max_len:
            ids = ids[-(max_len - 1):]
        rid = request_id or f"req-{self._next_seq}"
        gen = None
        if params.seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(params.seed)
        r = _Request(rid, prompt if isinstance(prompt, str) else "", ids, params,
                     RequestMetrics(rid, len(ids), 0, time.perf_counter()), self._next_seq, generator=gen)
        self._next_seq += 1
        self.waiting.append(r)
        return r

    def load_adapters(self, adapters: dict[str, dict[str, torch.Tensor]]) -> None:
        """Make named LoRA adapters available to requests (`GenerationParams.lora_name`).  The model must carry LoRA
        modules of matching shapes (`lora.get_peft_model`); requests that use different adapters, or none, are batched
        together (`multi_lora.BatchedLoRA`)."""
        from .multi_lora import BatchedLoRA
        limit = getattr(getattr(self.config, "lora", None), "max_loras", None)
        if limit and len(adapters) > limit:
            raise ValueError(f"{len(adapters)} adapters exceed lora.max_loras = {limit}")
        self.runner.lora = BatchedLoRA(self.model, adapters)
        self.adapter_states = dict(adapters)

    def _salt(self, r: "_Request") -> bytes:
        """Prefix-cache namespace of a request: K/V computed under one adapter are not valid under another."""
        name = r.params.lora_name if self.runner.lora is not None else None
        return b"" if name is None else b"lora:" + name.encode()

    def abort(self, request_id: str) -> bool:
        for q in (self.waiting, self.running):
            for r in list(q):
                if r.request_id == request_id:
                    q.remove(r)
                    self._finish(r, "abort")
                    return True
        return False

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def _finish(self, r: _Request, reason: str) -> None:
        r.finished, r.finish_reason = True, reason
        r.metrics.finished = time.perf_counter()
        r.metrics.completion_tokens = len(r.output_ids)
        self.cache.register_full_blocks(r.seq_id, r.prompt_ids + r.output_ids, self._salt(r)) if r.seq_id in self.cache.seqs else None
        self.cache.free_sequence(r.seq_id)
        if self.config.observability.collect_metrics:
            self.metrics.add(r.metrics)

    # -------------------------------------------------------------- one engine step
    def step(self) -> list[tuple[_Request, int]]:
        """Runs one forward over the scheduled tokens; returns (request, new token) for every request that sampled."""
        sc = self.config.scheduler
        budget = sc.max_num_batched_tokens
        batch: list[tuple[_Request, list[int], int]] = []   # (request, tokens fed this step, start position)
        # 1) decode tokens of running requests
        for r in list(self.running):
            if budget <= 0:
                break
            if not self.cache.can_append(r.seq_id, 1):
                # out of blocks: preempt the most recent request (recompute later)
                self.running.remove(r)
                self.cache.free_sequence(r.seq_id)
                r.prefilled = 0
                r.prompt_ids = r.prompt_ids + r.output_ids
                self.waiting.appendleft(r)
                continue
            if r.prefilled < len(r.prompt_ids):
                continue
            batch.append((r, [r.output_ids[-1]], len(r.prompt_ids) + len(r.output_ids) - 1))
            budget -= 1
        # 2) (chunked) prefill
        candidates = [r for r in self.running if r.prefilled < len(r.prompt_ids)]
        while self.waiting and len(self.running) < sc.max_num_seqs:
            r = self.waiting.popleft()
            if r.prefilled == 0:
                covered = self.cache.match_prefix(r.seq_id, r.prompt_ids, self._salt(r))
                r.prefilled = covered
                r.metrics.cached_prompt_tokens = covered
            self.running.append(r)
            candidates.append(r)
        for r in candidates:
            if budget <= 0:
                break
            remaining = len(r.prompt_ids) - r.prefilled
            n = min(remaining, budget) if sc.enable_chunked_prefill else remaining
            if n <= 0 or (not sc.enable_chunked_prefill and n > budget and batch):
                continue
            if not self.cache.can_append(r.seq_id, n):
                continue
            batch.append((r, r.prompt_ids[r.prefilled:r.prefilled + n], r.prefilled))
            budget -= n
        if not batch:
            return []
        # 3) build the flattened inputs
        toks, pos, slots, seq_ids, q_lens, ad = [], [], [], [], [], []
        fresh = True
        lora = self.runner.lora
        for r, feed, start in batch:
            s = self.cache.append_slots(r.seq_id, len(feed))
            toks += feed
            if lora is not None:
                ad += lora.ids_for([r.params.lora_name]) * len(feed)
            pos += list(range(start, start + len(feed)))
            slots += s
            seq_ids.append(r.seq_id)
            q_lens.append(len(feed))
            fresh &= (start == 0)
        dev = self.device
        graphed = self.runner.can_graph(q_lens)
        if graphed:
            all_logits = self.runner.decode_graphed(toks, pos, slots, seq_ids)     # [n, V] of every decode row
            hidden = None
        else:
            hidden = self.runner.forward(torch.tensor(toks, device=dev), torch.tensor(pos, device=dev),
                                         torch.tensor(slots, device=dev, dtype=torch.long), seq_ids, q_lens, fresh,
                                         torch.tensor(ad, device=dev) if lora is not None else None)
        self.steps += 1
        # 4) sample for every request whose prompt is now complete
        sample_rows, sample_reqs = [], []
        for i, (r, feed, start) in enumerate(batch):
            if start + len(feed) >= len(r.prompt_ids):
                if r.prefilled < len(r.prompt_ids):
                    r.prefilled = len(r.prompt_ids)
                    self.cache.register_full_blocks(r.seq_id, r.prompt_ids, self._salt(r))
                sample_rows.append(i)
                sample_reqs.append(r)
            else:
                r.prefilled = start + len(feed)
        if not sample_reqs:
            return []
        rows = torch.tensor(sample_rows, device=dev)
        logits = all_logits[rows] if graphed else self.runner.logits(hidden[rows])
        ps = [r.params for r in sample_reqs]
        logits = apply_penalties(logits, [r.output_ids for r in sample_reqs], [p.repetition_penalty for p in ps],
                                 [p.presence_penalty for p in ps], [p.frequency_penalty for p in ps])
        ids, lps = sample(logits, [p.temperature for p in ps], [p.top_k for p in ps], [p.top_p for p in ps],
                          [p.min_p for p in ps], [r.generator for r in sample_reqs])
        now = time.perf_counter()
        out = []
        eos = self.tokenizer.eos_token_id
        for r, t, lp in zip(sample_reqs, ids.tolist(), lps.tolist()):
            r.output_ids.append(t)
            if r.params.logprobs:
                r.logprobs.append(lp)
            if r.metrics.first_token is None:
                r.metrics.first_token = now
            out.append((r, t))
            reason = None
            if (t == eos and not r.params.ignore_eos) or t in r.params.stop_token_ids:
                reason = "stop"
            elif len(r.output_ids) >= r.params.max_tokens or \
                    len(r.prompt_ids) + len(r.output_ids) >= self.config.cache.max_model_len:
                reason = "length"
            elif r.params.stop:
                text = self.tokenizer.decode(r.output_ids)
                if any(s in text for s in r.params.stop):
                    reason = "stop"
            if reason:
                self.running.remove(r)
                self._finish(r, reason)
        return out

    def decode_text(self, r: _Request) -> str:
        ids = r.output_ids
        if ids and r.finish_reason == "stop" and ids[-1] == self.tokenizer.eos_token_id:
            ids = ids[:-1]
        text = self.tokenizer.decode(ids)
        for s in r.params.stop:
            if s in text:
                text = text[:text.index(s)]
        return text


def _lora_request_parts(req) -> tuple[str, str | None]:
    """(adapter name, adapter directory or None) from a name, a mapping or an object with `lora_name` / `lora_path`."""
    if isinstance(req, str):
        return req, None
    get = req.get if isinstance(req, dict) else (lambda k, d=None: getattr(req, k, d))
    return get("lora_name"), get("lora_path", None)


class EngineBuilder:
    def __init__(self, config: EngineConfig | None = None):
        self.config = config or EngineConfig()

    def build_sync(self, model=None, tokenizer=None, *, config: EngineConfig | None = None) -> "SOTAInferenceEngine":
        """`config` replaces the builder's own configuration for this engine (a config in the first position works
        too: `EngineBuilder().build_sync(config)`)."""
        if isinstance(model, EngineConfig):
            config, model = model, None
        return SOTAInferenceEngine(config or self.config, model, tokenizer)

    def build_async(self, model=None, tokenizer=None, *, config: EngineConfig | None = None) -> "SOTAAsyncStreamEngine":
        if isinstance(model, EngineConfig):
            config, model = model, None
        return SOTAAsyncStreamEngine(config or self.config, model, tokenizer)


class SOTAInferenceEngine:
    def __init__(self, config: EngineConfig | None = None, model=None, tokenizer=None, draft_model=None):
        self.config = config or EngineConfig()
        self.core = EngineCore(self.config, model, tokenizer)
        self.draft_model = draft_model      # small model of the same vocabulary for `speculative.enabled`

    def _generate_speculative(self, prompts: list[str], params: GenerationParams) -> list["InferenceResponse"]:
        """One request at a time through draft-and-verify decoding (inference/speculative.py)."""
        from .speculative import speculative_generate
        out = []
        for p in prompts:
            r = self.core.add_request(p, params)
            self.core.waiting.remove(r)
            gen = r.generator
            t0 = time.perf_counter()
            ids, stats = speculative_generate(self.core.model, self.draft_model, r.prompt_ids, params.max_tokens,
                                              k=self.config.speculative.num_speculative_tokens,
                                              temperature=params.temperature, eos_token_id=self.core.tokenizer.eos_token_id,
                                              generator=gen)
            r.output_ids = ids
            r.finish_reason = "stop" if ids and ids[-1] == self.core.tokenizer.eos_token_id else "length"
            r.metrics.completion_tokens = len(ids)
            r.metrics.first_token = t0
            r.metrics.finished = time.perf_counter()
            self.core.metrics.add(r.metrics)
            resp = InferenceResponse(r.request_id, r.prompt, self.core.decode_text(r), list(ids), r.finish_reason, r.metrics,
                                     None)
            resp.speculative_acceptance = stats.acceptance_rate
            out.append(resp)
        return out

    def generate(self, prompts: str | Iterable[str], params: GenerationParams | None = None, lora_request=None) -> Result:
        """`lora_request`: {"lora_name": ..., "lora_path": ...} (or an object with those attributes, or just the name
        of a loaded adapter): the adapter is loaded on first use and applied to these prompts."""
        if lora_request is not None:
            name, path = _lora_request_parts(lora_request)
            return self.generate_with_lora(prompts, name, path, params=params)
        try:
            single = isinstance(prompts, str)
            if self.config.speculative.enabled and self.draft_model is not None:
                res = self._generate_speculative([prompts] if single else list(prompts), params or GenerationParams())
                return Ok(res[0] if single else res)
            reqs = [self.core.add_request(p, params) for p in ([prompts] if single else list(prompts))]
            while self.core.has_unfinished():
                self.core.step()
            res = [InferenceResponse(r.request_id, r.prompt, self.core.decode_text(r), list(r.output_ids),
                                     r.finish_reason or "stop", r.metrics, r.logprobs or None) for r in reqs]
            return Ok(res[0] if single else res)
        except (ValueError, MemoryError, RuntimeError) as e:
            return Err(e)

    def metrics_summary(self) -> dict:
        return self.core.metrics.summary()

    get_metrics_summary = metrics_summary

    @property
    def engine(self) -> "EngineCore":
        """The scheduler / model-runner core (what the reference exposes as its underlying LLM engine)."""
        return self.core

    @property
    def metrics(self) -> "MetricsAggregator":
        return self.core.metrics

    def generate_single(self, prompt: str, params: GenerationParams | None = None, lora_request=None) -> Result:
        return self.generate(prompt, params, lora_request)

    def generate_with_lora(self, prompts: str | Iterable[str], lora_name: str, lora_path: str | None = None,
                           lora_id: int | None = None, params: GenerationParams | None = None) -> Result:
        """Generate with the named adapter.  `lora_path`: a directory written by `lora.save_adapter`, loaded on first
        use; adapters registered earlier with `EngineCore.load_adapters` are found by name alone."""
        import copy as _copy
        try:
            known = self.core.adapter_states
            if lora_name not in known:
                if lora_path is None:
                    raise ValueError(f"adapter {lora_name!r} is not loaded and no lora_path was given")
                from ..lora import adapter_state_from_dir
                self.core.load_adapters({**known, lora_name: adapter_state_from_dir(self.core.model, lora_path)})
        except (ValueError, OSError, RuntimeError, KeyError) as e:
            return Err(e)
        p = _copy.copy(params) if params is not None else GenerationParams()
        p.lora_name = lora_name
        return self.generate(prompts, p)


class SOTAAsyncStreamEngine:
    """Single background loop stepping the core; each request gets an asyncio queue of StreamChunks."""

    def __init__(self, config: EngineConfig | None = None, model=None, tokenizer=None):
        self.config = config or EngineConfig()
        self.core = EngineCore(self.config, model, tokenizer)
        self._queues: dict[str, asyncio.Queue] = {}
        self._task: asyncio.Task | None = None

    async def _loop(self):
        while self.core.has_unfinished():
            produced = await asyncio.get_running_loop().run_in_executor(None, self.core.step)
            for r, tok in produced:
                q = self._queues.get(r.request_id)
                if q is None:
                    continue
                full = self.core.decode_text(r)
                delta, r.emitted_text_len = full[r.emitted_text_len:], len(full)
                await q.put(StreamChunk(r.request_id, delta, tok, r.finished, r.finish_reason))
            await asyncio.sleep(0)
        self._task = None

    async def generate_stream(self, prompt: str, params: GenerationParams | None = None,
                              request_id: str | None = None, lora_request=None) -> AsyncIterator[StreamChunk]:
        if lora_request is not None:
            import copy as _copy
            name, path = _lora_request_parts(lora_request)
            if name not in self.core.adapter_states:
                if path is None:
                    raise ValueError(f"adapter {name!r} is not loaded and the request names no lora_path")
                from ..lora import adapter_state_from_dir
                self.core.load_adapters({**self.core.adapter_states, name: adapter_state_from_dir(self.core.model, path)})
            params = _copy.copy(params) if params is not None else GenerationParams()
            params.lora_name = name
        r = self.core.add_request(prompt, params, request_id)
        q: asyncio.Queue = asyncio.Queue()
        self._queues[r.request_id] = q
        if self._task is None:
            self._task = asyncio.create_task(self._loop())
        try:
            while True:
                chunk = await q.get()
                yield chunk
                if chunk.finished:
                    break
        finally:
            self._queues.pop(r.request_id, None)

    async def abort_request(self, request_id: str) -> bool:
        ok = self.core.abort(request_id)
        q = self._queues.get(request_id)
        if q is not None:
            await q.put(StreamChunk(request_id, "", -1, True, "abort"))
        return ok

    @property
    def engine(self) -> "EngineCore":
        return self.core

    @property
    def active_request_count(self) -> int:
        return len(self._queues)

    async def generate(self, prompt: str, params: GenerationParams | None = None, request_id: str | None = None,
                       lora_request=None) -> Result:
        """Non-streaming form: runs the streaming path and returns the whole completion."""
        try:
            text, ids, reason, rid = [], [], None, request_id
            async for c in self.generate_stream(prompt, params, request_id, lora_request):
                rid = c.request_id
                text.append(c.text)
                if c.token_id is not None and c.token_id >= 0:
                    ids.append(c.token_id)
                reason = c.finish_reason or reason
            m = next((x for x in reversed(self.core.metrics.records) if x.request_id == rid), RequestMetrics(rid or ""))
            return Ok(InferenceResponse(rid or "", prompt, "".join(text), ids, reason or "stop", m, None))
        except (ValueError, MemoryError, RuntimeError) as e:
            return Err(e)

    async def generate_batch(self, prompts: list[str], params: GenerationParams | None = None) -> Result:
        """All prompts are queued at once, so the scheduler batches them continuously."""
        results = await asyncio.gather(*(self.generate(p, params) for p in prompts))
        bad = next((r for r in results if r.is_err()), None)
        return bad if bad is not None else Ok([r.unwrap() for r in results])

    async def shutdown(self) -> None:
        for rid in list(self._queues):
            await self.abort_request(rid)
        if self._task is not None:
            try:
                await self._task
            except Exception:   # noqa: BLE001 - the loop ends with the aborted requests
                pass
        self._queues.clear()

    def get_metrics_summary(self) -> dict:
        out = self.core.metrics.summary()
        out["active_requests"] = self.active_request_count
        return out


class EnginePresets:
    @staticmethod
    def low_latency(model: str = "tiny") -> EngineConfig:
        return EngineConfig(model=model, scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=2048))

    @staticmethod
    def high_throughput(model: str = "tiny") -> EngineConfig:
        return EngineConfig(model=model, scheduler=SchedulerConfig(max_num_seqs=256, max_num_batched_tokens=16384))

    # ---- deployment profiles under the reference's names (data_pipeline/trainer/inference.py:1549-1810)
    @staticmethod
    def _base(model, tp_size, pp_size, max_model_len, seqs, tokens, util, chunked=True) -> EngineConfig:
        return EngineConfig(model=model, enforce_eager=False,
                            scheduler=SchedulerConfig(max_num_seqs=seqs, max_num_batched_tokens=tokens,
                                                      enable_chunked_prefill=chunked),
                            cache=CacheConfig(gpu_memory_utilization=util, enable_prefix_caching=True,
                                              max_model_len=max_model_len),
                            parallel=ParallelConfig(tensor_parallel_size=tp_size, pipeline_parallel_size=pp_size))

    @staticmethod
    def high_throughput_batch(model: str = "tiny", tp_size: int = 1, max_model_len: int = 8192) -> EngineConfig:
        return EnginePresets._base(model, tp_size, 1, max_model_len, 256, 32768, 0.95)

    @staticmethod
    def low_latency_interactive(model: str = "tiny", tp_size: int = 1, max_model_len: int = 4096) -> EngineConfig:
        return EnginePresets._base(model, tp_size, 1, max_model_len, 32, 4096, 0.90)

    @staticmethod
    def speculative_fast_decode(model: str = "tiny", draft_model: str | None = None, tp_size: int = 1,
                                num_speculative_tokens: int = 5, max_model_len: int = 4096) -> EngineConfig:
        c = EnginePresets._base(model, tp_size, 1, max_model_len, 64, 8192, 0.90, chunked=False)
        c.speculative = SpeculativeConfig(enabled=True, draft_model=draft_model,
                                          num_speculative_tokens=num_speculative_tokens)
        return c

    @staticmethod
    def quantized_memory_efficient(model: str = "tiny", quant_method="fp8", bits: int = 8, tp_size: int = 1,
                                   max_model_len: int = 8192) -> EngineConfig:
        c = EnginePresets._base(model, tp_size, 1, max_model_len, 128, 16384, 0.92)
        c.quantization = QuantizationConfig(method=str(getattr(quant_method, "value", quant_method)))
        return c

    @staticmethod
    def multi_gpu_large_model(model: str = "tiny", tp_size: int = 4, pp_size: int = 1,
                              max_model_len: int = 16384) -> EngineConfig:
        return EnginePresets._base(model, tp_size, pp_size, max_model_len, 128, 16384, 0.92)

    @staticmethod
    def multi_lora_serving(model: str = "tiny", max_lora_rank: int = 64, max_concurrent_loras: int = 4,
                           tp_size: int = 1, max_model_len: int = 4096) -> EngineConfig:
        c = EnginePresets._base(model, tp_size, 1, max_model_len, 64, 8192, 0.88)
        c.lora = LoRAServingConfig(enabled=True, max_loras=max_concurrent_loras, max_lora_rank=max_lora_rank)
        return c

    @staticmethod
    def long_context(model: str = "tiny", max_len: int = 131072) -> EngineConfig:
        return EngineConfig(model=model, cache=CacheConfig(max_model_len=max_len, block_size=32),
                            scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=8192))


# ------------------------------------------------------------------------------------------------ HTTP server
def create_openai_server(engine: "SOTAAsyncStreamEngine | EngineConfig", model_name: str = "trainscale", *, config=None,
                         host: str | None = None, port: int | None = None):
    """FastAPI application with the OpenAI-style routes.  `engine` may be an `EngineConfig` (`config=` in the
    reference's spelling): the streaming engine is then built from it and the model's name is the served name.  `host`
    and `port` are kept on `app.state` for whoever starts the server (`uvicorn.run(app, host=..., port=...)`)."""
    if config is not None or isinstance(engine, EngineConfig):
        cfg = config if config is not None else engine
        if isinstance(model_name, str) and host is None and model_name not in ("trainscale",) and "." in model_name:
            host, model_name = model_name, "trainscale"     # positional (config, host, port)
        engine = SOTAAsyncStreamEngine(cfg)
        model_name = cfg.model if model_name == "trainscale" else model_name
    from fastapi import FastAPI
    from fastapi.responses import PlainTextResponse, StreamingResponse
    from pydantic import BaseModel

    app = FastAPI(title="trainscale-b200 inference")

    class CompletionRequest(BaseModel):
        model: str | None = None
        prompt: str | list[str] = ""
        max_tokens: int = 128
        temperature: float = 0.7
        top_p: float = 1.0
        stop: list[str] | str | None = None
        stream: bool = False
        seed: int | None = None

    class ChatMessage(BaseModel):
        role: str
        content: str

    class ChatRequest(BaseModel):
        model: str | None = None
        messages: list[ChatMessage]
        max_tokens: int = 128
        temperature: float = 0.7
        top_p: float = 1.0
        stop: list[str] | str | None = None
        stream: bool = False
        seed: int | None = None

    def to_params(req) -> GenerationParams:
        stop = [req.stop] if isinstance(req.stop, str) else (req.stop or [])
        return GenerationParams(max_tokens=req.max_tokens, temperature=req.temperature, top_p=req.top_p, stop=stop,
                                seed=req.seed)

    async def run(prompt: str, params: GenerationParams):
        text, reason, n = "", "stop", 0
        async for ch in engine.generate_stream(prompt, params):
            text += ch.text
            n += 1
            reason = ch.finish_reason or reason
        return text, reason, n

    @app.get("/health")
    async def health():
        return {"status": "ok", "running": len(engine.core.running), "waiting": len(engine.core.waiting)}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(engine.core.metrics.prometheus())

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model"}]}

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest):
        params = to_params(req)
        prompt = req.prompt if isinstance(req.prompt, str) else req.prompt[0]
        if req.stream:
            async def gen():
                async for ch in engine.generate_stream(prompt, params):
                    yield "data: " + json.dumps({"object": "text_completion", "model": model_name,
                                                 "choices": [{"index": 0, "text": ch.text,
                                                              "finish_reason": ch.finish_reason}]}) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        text, reason, n = await run(prompt, params)
        return {"object": "text_completion", "model": model_name,
                "choices": [{"index": 0, "text": text, "finish_reason": reason}],
                "usage": {"completion_tokens": n}}

    @app.post("/v1/chat/completions")
    async def chat(req: ChatRequest):
        params = to_params(req)
        prompt = engine.core.tokenizer.apply_chat_template([m.model_dump() for m in req.messages], True)
        if req.stream:
            async def gen():
                async for ch in engine.generate_stream(prompt, params):
                    yield "data: " + json.dumps({"object": "chat.completion.chunk", "model": model_name,
                                                 "choices": [{"index": 0, "delta": {"content": ch.text},
                                                              "finish_reason": ch.finish_reason}]}) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        text, reason, n = await run(prompt, params)
        return {"object": "chat.completion", "model": model_name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": reason}],
                "usage": {"completion_tokens": n}}

    app.state.host, app.state.port = host or "0.0.0.0", int(port or 8000)
    return app


# ------------------------------------------------------------------------------------------------ CLI
def run_bench(engine: SOTAInferenceEngine, num_prompts: int = 50, input_len: int = 128, output_len: int = 128,
              warmup: bool = True) -> dict:
    """Offline throughput / latency of the engine on random prompts (all requests arrive at t = 0): TTFT and TPOT
    percentiles from the per-request metrics, output and total tokens per second over the whole run.  A short warm-up
    with the same batch shape runs first, so that library loading and CUDA-graph capture are not in the numbers."""
    vocab = min(engine.core.model.config.vocab_size, 255)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(1, vocab, (input_len,), generator=g).tolist() for _ in range(num_prompts)]
    params = GenerationParams(max_tokens=output_len, temperature=0.0, ignore_eos=True)
    if warmup:
        wp = GenerationParams(max_tokens=min(8, output_len), temperature=0.0, ignore_eos=True)
        for p in prompts:
            engine.core.add_request([t % vocab + 1 for t in p[::-1]], wp)      # other tokens: no prefix-cache hits later
        while engine.core.has_unfinished():
            engine.core.step()
        engine.core.metrics = MetricsAggregator()
        engine.core.steps = 0
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        engine.core.add_request(p, params)
    while engine.core.has_unfinished():
        engine.core.step()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    s = engine.metrics_summary()
    s.update(seconds=dt, output_tokens_per_second=num_prompts * output_len / dt,
             total_tokens_per_second=num_prompts * (input_len + output_len) / dt, engine_steps=engine.core.steps,
             cuda_graph_replays=engine.core.runner.graph_replays, cuda_graphs=len(engine.core.runner.graphs),
             tensor_parallel_size=engine.core.config.parallel.tensor_parallel_size)
    return s


def run_hf_generate_baseline(model_cfg, num_prompts: int, input_len: int, output_len: int, batch_size: int = 64) -> dict:
    """The same workload through HuggingFace `generate` on a random-init model of the same shape (the path the
    reference's engine falls back to without vLLM, data_pipeline/trainer/inference.py:2177-2233): bf16, SDPA
    attention, greedy, static batches of `batch_size` prompts.  TTFT = time of a 1-token generate of a batch
    (prefill), TPOT = (full generate - prefill) / (output_len - 1)."""
    from transformers import LlamaConfig as HFConfig, LlamaForCausalLM as HFModel
    c = model_cfg
    hf = HFConfig(vocab_size=c.vocab_size, hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
                  num_hidden_layers=c.num_hidden_layers, num_attention_heads=c.num_attention_heads,
                  num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim, rms_norm_eps=c.rms_norm_eps,
                  rope_theta=c.rope_theta, max_position_embeddings=max(c.max_position_embeddings, input_len + output_len),
                  tie_word_embeddings=c.tie_word_embeddings, attn_implementation="sdpa")
    torch.manual_seed(0)
    with torch.device("cuda"):
        m = HFModel(hf).to(torch.bfloat16).eval()
    vocab = min(c.vocab_size, 255)
    g = torch.Generator().manual_seed(0)
    ids = torch.stack([torch.randint(1, vocab, (input_len,), generator=g) for _ in range(num_prompts)]).cuda()
    kw = dict(do_sample=False, pad_token_id=0, eos_token_id=None)
    with torch.no_grad():
        m.generate(ids[:min(batch_size, 4)], max_new_tokens=4, min_new_tokens=4, **kw)     # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        m.generate(ids[:batch_size], max_new_tokens=1, min_new_tokens=1, **kw)
        torch.cuda.synchronize()
        ttft = time.perf_counter() - t0
        t0 = time.perf_counter()
        for s0 in range(0, num_prompts, batch_size):
            m.generate(ids[s0:s0 + batch_size], max_new_tokens=output_len, min_new_tokens=output_len, **kw)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    nb = -(-num_prompts // batch_size)
    return {"impl": "transformers generate (bf16, sdpa)", "seconds": dt, "batch_size": batch_size,
            "output_tokens_per_second": num_prompts * output_len / dt,
            "total_tokens_per_second": num_prompts * (input_len + output_len) / dt,
            "ttft_first_batch_s": ttft, "tpot_s": max(0.0, dt / nb - ttft) / max(1, output_len - 1)}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m trainscale_b200.inference")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("probe", "batch", "stream", "serve", "bench"):
        p = sub.add_parser(name)
        p.add_argument("--model", default="tiny")
        p.add_argument("--max-tokens", type=int, default=64)
        p.add_argument("--temperature", type=float, default=0.7)
        if name in ("batch", "stream"):
            p.add_argument("--prompt", action="append", default=[])
        if name == "serve":
            p.add_argument("--host", default="127.0.0.1")
            p.add_argument("--port", type=int, default=8000)
        if name == "bench":
            p.add_argument("--num-prompts", type=int, default=50)
            p.add_argument("--input-len", type=int, default=128)
            p.add_argument("--output-len", type=int, default=128)
            p.add_argument("--baseline", default=None, choices=["hf"], help="also time transformers generate")
        p.add_argument("--tensor-parallel-size", type=int, default=1, help="launch under torchrun with this many ranks")
        p.add_argument("--eager", action="store_true", help="no CUDA graphs in the decode loop")
        p.add_argument("--max-num-seqs", type=int, default=64)
    a = ap.parse_args(argv)
    cfg = EngineConfig(model=a.model, enforce_eager=a.eager)
    cfg.parallel.tensor_parallel_size = a.tensor_parallel_size
    cfg.scheduler.max_num_seqs = a.max_num_seqs
    rank0 = True
    if a.tensor_parallel_size > 1:
        import os

        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            cfg.device = f"cuda:{local}"
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
        rank0 = dist.get_rank() == 0
    if a.cmd == "probe":
        print(json.dumps({"cuda": torch.cuda.is_available(),
                          "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu",
                          "config": asdict(cfg)}, indent=2))
        return 0
    params = GenerationParams(max_tokens=a.max_tokens, temperature=a.temperature)
    if a.cmd == "batch":
        eng = SOTAInferenceEngine(cfg)
        for r in eng.generate(a.prompt or ["Hello"], params).unwrap():
            print(json.dumps({"prompt": r.prompt, "text": r.text, "finish_reason": r.finish_reason}))
        return 0
    if a.cmd == "stream":
        async def go():
            eng = SOTAAsyncStreamEngine(cfg)
            async for ch in eng.generate_stream((a.prompt or ["Hello"])[0], params):
                sys.stdout.write(ch.text)
                sys.stdout.flush()
            print()
        asyncio.run(go())
        return 0
    if a.cmd == "serve":
        import uvicorn
        uvicorn.run(create_openai_server(SOTAAsyncStreamEngine(cfg), a.model), host=a.host, port=a.port)
        return 0
    if a.cmd == "bench":
        eng = SOTAInferenceEngine(cfg)
        out = run_bench(eng, a.num_prompts, a.input_len, a.output_len)
        if a.baseline == "hf" and rank0 and torch.cuda.is_available():
            mcfg = eng.core.model.config
            del eng
            torch.cuda.empty_cache()
            out["baseline"] = run_hf_generate_baseline(mcfg, a.num_prompts, a.input_len, a.output_len, a.max_num_seqs)
        if rank0:
            print(json.dumps(out))
        return 0
    return 1


# ------------------------------------------------------------------------------------------------ reference surface
from enum import Enum  # noqa: E402


class QuantizationMethod(Enum):
    """Weight formats a serving engine may be asked for (data_pipeline/trainer/inference.py:184).  This engine serves
    bf16 and block-scaled fp8; the others are accepted in configurations and refused at build time."""
    NONE = "none"
    GPTQ = "gptq"
    AWQ = "awq"
    AUTOROUND = "autoround"
    FP8 = "fp8"
    INT8 = "compressed-tensors"
    BITSANDBYTES = "bitsandbytes"
    SQUEEZELLM = "squeezellm"
    MARLIN = "marlin"


class ParallelStrategy(Enum):
    NONE = "none"
    TENSOR = "tensor"
    PIPELINE = "pipeline"
    TENSOR_PIPELINE = "tensor_pipeline"
    DATA = "data"


class SchedulerPolicy(Enum):
    FCFS = "fcfs"
    PRIORITY = "priority"


class ResultStatus(Enum):
    OK = "ok"
    ERR = "err"

    @classmethod
    def of(cls, result) -> "ResultStatus":
        return cls.OK if result.is_ok() else cls.ERR


@dataclass
class InferenceRequest:
    """A prompt with its sampling parameters, optional adapter and metrics; `submit(engine)` queues it."""
    prompt: str
    request_id: str = ""
    params: GenerationParams = field(default_factory=GenerationParams)
    lora_name: str | None = None
    lora_path: str | None = None
    lora_id: int | None = None
    _metrics: RequestMetrics = field(default_factory=RequestMetrics)

    def __post_init__(self):
        if not self.request_id:
            import uuid
            self.request_id = uuid.uuid4().hex
        self._metrics.request_id = self.request_id
        if self.lora_name and not self.params.lora_name:
            self.params.lora_name = self.lora_name

    @property
    def metrics(self) -> RequestMetrics:
        return self._metrics

    def get_lora_request(self) -> dict | None:
        """{"lora_name", "lora_int_id", "lora_path"} when the request names an adapter completely, else None."""
        if self.lora_name and self.lora_path and self.lora_id is not None:
            return {"lora_name": self.lora_name, "lora_int_id": self.lora_id, "lora_path": self.lora_path}
        return None

    def submit(self, engine: "SOTAInferenceEngine"):
        req = engine.core.add_request(self.prompt, self.params)
        self._metrics = req.metrics
        return req


class HardwareProbe:
    """What the serving engine can count on: devices, memory, compute capability, peer access, the dtype and attention
    path it will pick (data_pipeline/trainer/inference.py:702)."""

    @staticmethod
    def probe() -> dict:
        info: dict = {"cuda_available": torch.cuda.is_available(), "gpu_count": 0, "devices": [],
                      "total_gpu_memory_gb": 0.0, "recommended_dtype": "float32", "recommended_attention": "reference",
                      "nvlink_p2p": False}
        if not torch.cuda.is_available():
            return info
        n = torch.cuda.device_count()
        info["gpu_count"] = n
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            info["devices"].append({"index": i, "name": p.name, "compute_capability": f"{p.major}.{p.minor}",
                                    "memory_gb": round(p.total_memory / 2 ** 30, 1), "sm_count": p.multi_processor_count})
            info["total_gpu_memory_gb"] += p.total_memory / 2 ** 30
        major = torch.cuda.get_device_capability(0)[0]
        info["recommended_dtype"] = "bfloat16" if major >= 8 else "float16"
        info["recommended_attention"] = "tcgen05_flash" if major == 10 else "reference"
        info["cuda_graphs"] = True
        if n > 1:
            try:
                info["nvlink_p2p"] = all(torch.cuda.can_device_access_peer(0, j) for j in range(1, n))
            except RuntimeError:
                pass
        info["recommended_tensor_parallel_size"] = n if info["nvlink_p2p"] else 1
        return info


def run_hardware_probe() -> dict:
    info = HardwareProbe.probe()
    print(json.dumps(info, indent=2))
    return info


def run_batch_demo(config: EngineConfig, prompts: list[str], params: GenerationParams | None = None) -> list:
    """Generate for a batch of prompts and print every completion with its latency figures and the engine summary."""
    engine = SOTAInferenceEngine(config)
    params = params or GenerationParams(max_tokens=256, temperature=0.7, top_p=0.95)
    responses = engine.generate(list(prompts), params).unwrap()
    for r in responses:
        m = r.metrics
        print(f"[{r.request_id[:8]}] {r.finish_reason:6s} {m.completion_tokens:4d} tok  {r.text!r}")
    print(json.dumps(engine.metrics_summary(), indent=2, default=str))
    return responses


def run_benchmark(config: EngineConfig, num_prompts: int = 100, prompt_len: int = 128, output_len: int = 128) -> dict:
    """Throughput and TTFT / TPOT percentiles of an engine built from `config` (`run_bench` on a fresh engine)."""
    out = run_bench(SOTAInferenceEngine(config), num_prompts, prompt_len, output_len)
    print(json.dumps(out, indent=2, default=str))
    return out
