"""CUDA-graph capture of launch-bound loops (decode steps, fixed-shape micro-steps).

Stands in for the reference's torch.compile wrapper (data_pipeline/trainer/kernels/compiler.py:156-1066:
`CompilationConfig`, `CUDAGraphManager`, `compile_model`, `optimize_for_inference / training`): this framework has no
tracing compiler on the hot path - kernels are hand-written - so the only launch-overhead tool is graph replay.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from .refargs import ANY, reference_kwargs


@dataclass
class CompilationConfig:
    mode: str = "cuda_graphs"      # cuda_graphs | none
    warmup_iters: int = 3
    pool_shared: bool = True


class CUDAGraphManager:
    """Capture `fn(*static_inputs)` once per input-shape signature and replay it with new data copied in."""

    def __init__(self, config: CompilationConfig | None = None):
        self.config = config or CompilationConfig()
        self.graphs: dict[tuple, tuple] = {}
        self.pool = None

    @staticmethod
    def _sig(args) -> tuple:
        return tuple((tuple(a.shape), a.dtype) if torch.is_tensor(a) else a for a in args)

    def run(self, fn: Callable, *args):
        if not torch.cuda.is_available() or self.config.mode == "none":
            return fn(*args)
        sig = (id(fn),) + self._sig(args)
        if sig not in self.graphs:
            static = [a.clone() if torch.is_tensor(a) else a for a in args]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(self.config.warmup_iters):
                    fn(*static)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self.pool):
                out = fn(*static)
            if self.config.pool_shared and self.pool is None:
                self.pool = g.pool()
            self.graphs[sig] = (g, static, out)
        g, static, out = self.graphs[sig]
        for s_, a in zip(static, args):
            if torch.is_tensor(a):
                s_.copy_(a)
        g.replay()
        return out

    def clear(self):
        self.graphs.clear()
        self.pool = None
        self.__dict__.get("_keyed", {}).clear()

    # ---- explicit two-step form (data_pipeline/trainer/kernels/compiler.py:308-400)
    def capture(self, func: Callable, *args: torch.Tensor, key: str | None = None, **kwargs):
        """Capture `func(*args, **kwargs)` under `key` (default: the function's identity).  Returns (graph, static
        inputs, static outputs); a second call with the same key returns the stored triple.  Needs a CUDA device."""
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA required for graph capture")
        keyed = self.__dict__.setdefault("_keyed", {})
        key = key or str(id(func))
        if key in keyed:
            return keyed[key]
        static = [a.clone() for a in args if torch.is_tensor(a)]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(self.config.warmup_iters):
                func(*static, **kwargs)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=self.pool):
            out = func(*static, **kwargs)
        if self.config.pool_shared and self.pool is None:
            self.pool = g.pool()
        outs = [out] if torch.is_tensor(out) else [o for o in out if torch.is_tensor(o)]
        keyed[key] = (g, static, outs)
        return keyed[key]

    def replay(self, key: str, *args: torch.Tensor):
        """Copy `args` into the static inputs of the graph captured under `key`, replay it, and return its static
        outputs (one tensor, or a list).  The outputs are overwritten by the next replay: clone what must be kept."""
        keyed = self.__dict__.get("_keyed", {})
        if key not in keyed:
            raise KeyError(f"no graph captured under {key!r}")
        g, static, outs = keyed[key]
        new = [a for a in args if torch.is_tensor(a)]
        if len(new) != len(static):
            raise ValueError(f"graph {key!r} takes {len(static)} tensors, got {len(new)}")
        for dst, src in zip(static, new):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise ValueError(f"graph {key!r} was captured for {tuple(dst.shape)} {dst.dtype}")
            dst.copy_(src)
        g.replay()
        return outs[0] if len(outs) == 1 else outs


_TRACER_OPTIONS = {"fullgraph": ANY, "dynamic": ANY, "mode": ANY, "backend": ANY, "example_inputs": ANY}


@reference_kwargs(_TRACER_OPTIONS)
def compile_model(model, config: CompilationConfig | None = None):
    """Returns a callable running `model` under graph replay for fixed input shapes (inference only).  The options of
    the reference's tracing compiler (`fullgraph`, `dynamic`, `mode`, `backend`, `example_inputs`) are accepted and
    have no counterpart here: kernels are hand-written, only launches are captured."""
    mgr = CUDAGraphManager(config)

    def call(*tensors):
        out = model(*tensors)
        return out.logits if hasattr(out, "logits") else out

    @torch.no_grad()
    def run(*args, input_ids=None):
        """`run(input_ids)` for a language model (its logits come back), or the positional tensors of any module."""
        return mgr.run(call, *(((input_ids,) if input_ids is not None else ()) + args))

    run.manager = mgr
    return run


@reference_kwargs({"example_inputs": ANY, "use_cudagraphs": (True, None), "use_channels_last": (False, None),
                   "freeze": (True, None)})
def optimize_for_inference(model):
    model.eval()
    for p in model.parameters():
        p.requires_grad_(False)
    return compile_model(model)


def optimize_for_training(model, checkpoint_every: int = 2, *, use_activation_checkpointing: bool = True):
    """Recompute every `checkpoint_every`-th layer in backward (`use_activation_checkpointing=False`: leave the model
    as it is)."""
    if use_activation_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
        model.gradient_checkpointing_enable(checkpoint_every)
    return model


class ModelCompiler:
    """Facade with the reference's compiler surface (data_pipeline/trainer/kernels/compiler.py:513) on this
    framework's mechanism: kernels are hand-written, so "compiling" a model means capturing its launch-bound step in a
    CUDA graph and choosing the recompute policy, not tracing it."""

    def __init__(self, config: CompilationConfig | None = None):
        self.config = config or CompilationConfig()
        self.graphs = CUDAGraphManager()

    def compile(self, model, example_inputs=None):
        """`example_inputs` (a tensor or a tuple of them): one call is made right away, so that the graph of that shape
        is captured here and not on the first training step."""
        compiled = compile_model(model, self.config)
        if example_inputs is not None:
            args = example_inputs if isinstance(example_inputs, (tuple, list)) else (example_inputs,)
            with torch.no_grad():
                compiled(*args)
        return compiled

    def for_inference(self, model):
        return optimize_for_inference(model)

    def for_training(self, model, checkpoint_every: int = 2):
        return optimize_for_training(model, checkpoint_every)

    @property
    def cuda_graph_manager(self) -> CUDAGraphManager:
        return self.graphs

    def reset(self) -> None:
        """Drop every captured graph (their memory pool with them)."""
        self.graphs.clear()


class InductorConfigManager:
    """The reference tunes TorchInductor through this class (data_pipeline/trainer/kernels/compiler.py:190-288:
    max-autotune, coordinate descent, epilogue fusion, CUDA-graph trees).  This framework has no tracing compiler on
    its hot path, so the manager keeps the same interface but only (a) records the requested options, (b) maps the one
    option that has a counterpart here - CUDA-graph capture - onto `CompilationConfig`, and (c) can apply the options
    to `torch._inductor.config` for USER code that calls `torch.compile` on modules outside the framework
    (`apply_to_torch=True`; restored by `restore()` / on leaving the `with` block)."""

    KNOWN = ("max_autotune", "max_autotune_gemm", "coordinate_descent_tuning", "epilogue_fusion", "triton.cudagraphs",
             "triton.cudagraph_trees", "shape_padding", "fx_graph_cache")

    def __init__(self, apply_to_torch: bool = False, **options):
        self.apply_to_torch = apply_to_torch
        self.options: dict[str, object] = {}
        self._saved: dict[str, object] = {}
        self.configure(**options)

    def configure(self, **options) -> "InductorConfigManager":
        for k, v in options.items():
            self.options[k.replace("__", ".")] = v
        return self

    def for_mode(self, mode: str) -> "InductorConfigManager":
        """default | reduce-overhead | max-autotune, as in `torch.compile(mode=...)`."""
        presets = {"default": {}, "reduce-overhead": {"triton.cudagraphs": True},
                   "max-autotune": {"max_autotune": True, "coordinate_descent_tuning": True, "triton.cudagraphs": True}}
        if mode not in presets:
            raise ValueError(f"unknown mode {mode!r}")
        self.options.update(presets[mode])
        return self

    def compilation_config(self) -> CompilationConfig:
        graphs = bool(self.options.get("triton.cudagraphs") or self.options.get("triton.cudagraph_trees"))
        return CompilationConfig(mode="cuda_graphs" if graphs else "none")

    def _target(self):
        try:
            import torch._inductor.config as cfg
            return cfg
        except Exception:
            return None

    _last: "InductorConfigManager | None" = None

    @classmethod
    def from_config(cls, config, apply_to_torch: bool = True) -> "InductorConfigManager":
        """Manager for an `InductorConfig` dataclass: `triton_x` fields become the `triton.x` options, `extra` is merged."""
        import dataclasses
        fields = dataclasses.asdict(config) if dataclasses.is_dataclass(config) else dict(config)
        extra = fields.pop("extra", None) or {}
        opts = {("triton." + k[len("triton_"):] if k.startswith("triton_") else k): v for k, v in fields.items()}
        opts.update(extra)
        m = cls(apply_to_torch=apply_to_torch)
        m.options.update(opts)
        return m

    def apply(self=None, config=None) -> dict[str, object]:
        """Returns the options that were actually set on torch's inductor config (empty unless apply_to_torch).
        `InductorConfigManager.apply(config)` on the CLASS is the reference's form: the `InductorConfig` is applied to
        torch's inductor settings (for user code that calls `torch.compile`), `InductorConfigManager.restore()` on the
        class undoes it."""
        if not isinstance(self, InductorConfigManager):
            config = config if config is not None else self
            InductorConfigManager._last = InductorConfigManager.from_config(config)
            return InductorConfigManager._last.apply()
        if config is not None:
            self.options.update(InductorConfigManager.from_config(config).options)
        done: dict[str, object] = {}
        cfg = self._target() if self.apply_to_torch else None
        if cfg is None:
            return done
        for k, v in self.options.items():
            obj, name = cfg, k
            if "." in k:
                head, name = k.split(".", 1)
                obj = getattr(cfg, head, None)
            if obj is not None and hasattr(obj, name):
                self._saved.setdefault(k, getattr(obj, name))
                setattr(obj, name, v)
                done[k] = v
        return done

    def restore(self=None) -> None:
        if not isinstance(self, InductorConfigManager):           # InductorConfigManager.restore() on the class
            if InductorConfigManager._last is not None:
                InductorConfigManager._last.restore()
            return
        cfg = self._target()
        if cfg is None:
            return
        for k, v in self._saved.items():
            obj, name = cfg, k
            if "." in k:
                head, name = k.split(".", 1)
                obj = getattr(cfg, head)
            setattr(obj, name, v)
        self._saved.clear()

    def __enter__(self):
        self.apply()
        return self

    def __exit__(self, *exc):
        self.restore()


# ------------------------------------------------------------------------------------------------ diagnostics
_STATS = {"captures": 0, "replays": 0, "eager_calls": 0, "signatures": 0}
_DEBUG = {"on": False}


def get_compilation_stats(manager: CUDAGraphManager | None = None) -> dict:
    """Counters of graph capture / replay (of one manager, or process-wide when none is given)."""
    if manager is not None:
        return {"signatures": len(manager.graphs), "pool_shared": manager.pool is not None,
                "captures": getattr(manager, "captures", len(manager.graphs)), "replays": getattr(manager, "replays", 0)}
    return dict(_STATS)


class compilation_debug_mode:
    """`with compilation_debug_mode():` logs every capture (shape signature) and counts replays / eager calls."""

    def __init__(self, log=print):
        self.log = log

    def __enter__(self):
        self._prev = (_DEBUG["on"], _DEBUG.get("log"))
        _DEBUG["on"], _DEBUG["log"] = True, self.log
        return self

    def __exit__(self, *exc):
        _DEBUG["on"], _DEBUG["log"] = self._prev


_orig_run = CUDAGraphManager.run


def _counted_run(self, fn, *args):
    if not torch.cuda.is_available() or self.config.mode == "none":
        _STATS["eager_calls"] += 1
        return _orig_run(self, fn, *args)
    before = len(self.graphs)
    out = _orig_run(self, fn, *args)
    if len(self.graphs) > before:
        _STATS["captures"] += 1
        _STATS["signatures"] += 1
        self.captures = getattr(self, "captures", 0) + 1
        if _DEBUG["on"]:
            _DEBUG["log"](f"[cuda-graph] captured {getattr(fn, '__name__', fn)} for {self._sig(args)}")
    _STATS["replays"] += 1
    self.replays = getattr(self, "replays", 0) + 1
    return out


CUDAGraphManager.run = _counted_run
