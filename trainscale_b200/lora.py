"""LoRA / rsLoRA / DoRA-style adapters for the framework decoder's fused projections.

Surface after data_pipeline/trainer/lora.py:69-408 (`LoRALinear`, `get_peft_model`, `merge_and_unload`, `apply_lora`)
and the fused LoRA kernels of data_pipeline/trainer/kernels/fast_lora_mlp.py:126-631: the adapter path
`s * (x A^T) B^T` runs on the tcgen05 GEMM next to the frozen base GEMM, and its backward is four small GEMMs.
HF target names (q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj) map onto row blocks of the fused
`wqkv` / `w_gate_up` weights, so a q/v-only LoRA touches only those output rows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from .ops import gemm
from .utils.refargs import ANY, reference_kwargs


class LoRALinear(nn.Module):
    """Low-rank update for one row block [row0, row0+rows) of a (possibly fused) weight."""

    def __init__(self, in_features: int, rows: int | None = None, r: int = 16, alpha: float = 32.0, dropout: float = 0.0,
                 use_rslora: bool | None = None, row0: int = 0, total_rows: int | None = None, dtype=None, device=None,
                 init: bool | str = True, bias: bool = False, *, out_features: int | None = None,
                 lora_alpha: float | None = None, lora_dropout: float | None = None):
        """`rows` is the adapter's output width.  `bias=True` adds a trainable output bias, used by the stand-alone
        form (`forward` with a base weight).  The reference's names `out_features`, `lora_alpha`, `lora_dropout` are
        taken as well; a layer built with them scales by alpha / r like the reference's (data_pipeline/trainer/lora.py:95)
        unless `use_rslora` is given, whereas this framework's default is the rank-stabilised alpha / sqrt(r)."""
        ref_form = out_features is not None or lora_alpha is not None
        rows = rows if rows is not None else out_features
        alpha = alpha if lora_alpha is None else lora_alpha
        dropout = dropout if lora_dropout is None else lora_dropout
        if use_rslora is None:
            use_rslora = not ref_form
        super().__init__()
        self._want_bias = bias
        self.r, self.row0, self.rows, self.total_rows = r, row0, rows, total_rows or rows
        self.scaling = alpha / math.sqrt(r) if use_rslora else alpha / r
        self.lora_A = nn.Parameter(torch.empty(r, in_features, dtype=dtype, device=device))
        self.lora_B = nn.Parameter(torch.zeros(rows, r, dtype=dtype, device=device))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        self._init = init
        self.weight = None            # frozen base weight: only when built by `from_linear` (stand-alone layer)
        self.bias_param = nn.Parameter(torch.zeros(rows, dtype=dtype, device=device)) if bias else None
        self.reset_lora_parameters()

    def reset_lora_parameters(self) -> None:
        """A: Kaiming-uniform (or N(0, 1/r) for init='gaussian'); B: zero, so the adapter starts as a no-op."""
        if self._init == "gaussian":
            nn.init.normal_(self.lora_A, std=1.0 / self.r)
        else:
            nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B)

    @classmethod
    def from_linear(cls, linear: nn.Linear, r: int = 16, lora_alpha: float = 32.0, lora_dropout: float = 0.0,
                    use_rslora: bool = False) -> "LoRALinear":
        """A stand-alone adapted layer around an existing nn.Linear, whose weight is shared and frozen
        (data_pipeline/trainer/lora.py:148-174)."""
        m = cls(linear.in_features, linear.out_features, r, lora_alpha, lora_dropout, use_rslora,
                dtype=linear.weight.dtype, device=linear.weight.device)
        m.weight = nn.Parameter(linear.weight.data, requires_grad=False)
        if linear.bias is not None:
            m.bias_param = nn.Parameter(linear.bias.data.clone())
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """y = x W^T (+ b) + scaling * (x A^T) B^T; without a base weight, the low-rank term alone."""
        if self.weight is None:
            return self.delta(x)
        y = gemm.linear(x, self.weight) + self.delta(x)
        return y if self.bias_param is None else y + self.bias_param

    def merge_weights(self) -> torch.Tensor:
        """W + scaling * B A, as a new tensor in the base weight's dtype."""
        if self.weight is None:
            raise ValueError("no base weight to merge into")
        return (self.weight.float() + self.delta_weight()).to(self.weight.dtype)

    def delta(self, x: torch.Tensor) -> torch.Tensor:
        if self.dropout is not None:
            x = self.dropout(x)
        return gemm.linear(gemm.linear(x, self.lora_A), self.lora_B) * self.scaling

    def delta_weight(self) -> torch.Tensor:
        return (self.lora_B.float() @ self.lora_A.float()) * self.scaling


class FusedLoRA(nn.Module):
    """All adapters of one fused weight; output is laid out like the fused projection's output."""

    def __init__(self, parts: list[LoRALinear]):
        super().__init__()
        self.parts = nn.ModuleList(parts)

    def linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Base projection and all adapters in one autograd node (adapter products accumulated in the GEMM epilogue).
        Adapter dropout needs its own input, so that case takes the two-step path."""
        if any(p.dropout is not None and self.training for p in self.parts) or any(p.row0 % 8 for p in self.parts):
            return gemm.linear(x, w) + self.forward(x)
        meta = tuple((float(p.scaling), int(p.row0), int(p.rows)) for p in self.parts)
        ab = [t for p in self.parts for t in (p.lora_A, p.lora_B)]
        return _LoRALinearFn.apply(x, w, meta, *ab)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        total = self.parts[0].total_rows
        if len(self.parts) == 1 and self.parts[0].rows == total:
            return self.parts[0].delta(x)
        out = x.new_zeros(*x.shape[:-1], total)
        for p in self.parts:
            out[..., p.row0:p.row0 + p.rows] = p.delta(x)
        return out


class _LoRALinearFn(torch.autograd.Function):
    """y = x W^T + sum_i s_i (x A_i^T) B_i^T written into the column block of adapter i, with the adapter products
    accumulated by the GEMM epilogue (alpha / accumulate) straight into y - no delta tensor, no separate add pass.
    Backward mirrors it: dx = dy W + sum_i s_i (dy_i B_i) A_i (accumulating GEMMs), dA_i = s_i (dy_i B_i)^T x,
    dB_i = s_i dy_i^T (x A_i^T).  Covers what the reference does with its fused LoRA kernels
    (data_pipeline/trainer/kernels/lora_kernels.py: forward, dA / dB / dx backward)."""

    @staticmethod
    def forward(ctx, x, w, meta, *ab):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        y = gemm.matmul_nt(x2, w)
        ts = []
        for i, (s, row0, rows) in enumerate(meta):
            A, B = ab[2 * i], ab[2 * i + 1]
            t = gemm.matmul_nt(x2, A)
            gemm.matmul_nt(t, B, out=y[:, row0:row0 + rows], accumulate=True, alpha=s)
            ts.append(t)
        ctx.save_for_backward(x2, w, *ab, *ts)
        ctx.meta, ctx.shape = meta, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        n = len(ctx.meta)
        saved = ctx.saved_tensors
        x2, w, ab, ts = saved[0], saved[1], saved[2:2 + 2 * n], saved[2 + 2 * n:]
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx = gemm.matmul_nn(dy2, w) if need_x else None
        dw = gemm.matmul_tn(dy2, x2, out_dtype=torch.float32).to(w.dtype) if need_w else None
        grads = []
        for i, (s, row0, rows) in enumerate(ctx.meta):
            A, B = ab[2 * i], ab[2 * i + 1]
            dyi = dy2[:, row0:row0 + rows]
            g = gemm.matmul_nn(dyi, B)                                   # [T, r]
            if need_x:
                gemm.matmul_nn(g, A, out=dx, accumulate=True, alpha=s)
            grads.append(gemm.matmul_tn(g, x2, alpha=s).to(A.dtype) if ctx.needs_input_grad[3 + 2 * i] else None)
            grads.append(gemm.matmul_tn(dyi, ts[i], alpha=s).to(B.dtype) if ctx.needs_input_grad[4 + 2 * i] else None)
        return (dx.view(ctx.shape) if need_x else None, dw, None, *grads)


def _targets_for(model_cfg) -> dict:
    """HF projection name -> (module kind, fused weight name, row0, rows)."""
    D, Hq, Hkv, I = model_cfg.head_dim, model_cfg.num_attention_heads, model_cfg.num_key_value_heads, model_cfg.intermediate_size
    H = model_cfg.hidden_size
    return {"q_proj": ("attn", "wqkv", 0, Hq * D), "k_proj": ("attn", "wqkv", Hq * D, Hkv * D),
            "v_proj": ("attn", "wqkv", (Hq + Hkv) * D, Hkv * D), "o_proj": ("attn", "wo", 0, H),
            "gate_proj": ("mlp", "w_gate_up", 0, I), "up_proj": ("mlp", "w_gate_up", I, I),
            "down_proj": ("mlp", "w_down", 0, H)}


@reference_kwargs(config="r")
def get_peft_model(model, r: int = 16, lora_alpha: float = 32.0, lora_dropout: float = 0.0,
                   target_modules: list[str] | None = None, use_rslora: bool = True, modules_to_save: list[str] | None = None,
                   init_lora_weights: bool | str = True, rank_pattern: dict | None = None):
    """Freeze the base weights and attach adapters. Returns the same model object.  `r` may also be a `LoraConfig`
    (the peft calling form `get_peft_model(model, config)`), whose fields then replace the keyword arguments."""
    if not isinstance(r, int):
        cfg = r
        r, lora_alpha, lora_dropout = cfg.r, cfg.lora_alpha, cfg.lora_dropout
        target_modules, use_rslora = list(cfg.target_modules), cfg.use_rslora
        init_lora_weights, rank_pattern = cfg.init_lora_weights, dict(cfg.rank_pattern) or None
        # embeddings and the head stay frozen unless the caller names them: a LoraConfig's default lists both
        modules_to_save = modules_to_save
    targets = _targets_for(model.config)
    wanted = [t for t in (target_modules or list(targets)) if t in targets]
    for p in model.parameters():
        p.requires_grad_(False)
    for li, layer in enumerate(model.model.layers):
        for kind, mod in (("attn", layer.self_attn), ("mlp", layer.mlp)):
            inner = getattr(mod, "inner", mod)
            if hasattr(inner, "router"):
                continue                      # expert weights are 3-D; adapters attach to the attention projections only
            by_weight: dict[str, list[LoRALinear]] = {}
            for t in wanted:
                k, wname, row0, rows = targets[t]
                if k != kind:
                    continue
                w = getattr(inner, wname)
                rank = (rank_pattern or {}).get(f"layers.{li}.{t}", (rank_pattern or {}).get(t, r))
                by_weight.setdefault(wname, []).append(
                    LoRALinear(w.shape[1], rows, rank, lora_alpha, lora_dropout, use_rslora, row0, w.shape[0], w.dtype,
                               w.device, init_lora_weights))
            if by_weight:
                inner.lora = nn.ModuleDict({k: FusedLoRA(v) for k, v in by_weight.items()})
    for name in modules_to_save or []:
        for n, p in model.named_parameters():
            if name in n or (name == "lm_head" and n == "lm_head"):
                p.requires_grad_(True)
    return model


@torch.no_grad()
def merge_and_unload(model):
    """Fold every adapter into its base weight and remove the adapters."""
    for layer in model.model.layers:
        for mod in (layer.self_attn, layer.mlp):
            inner = getattr(mod, "inner", mod)
            if inner.lora is None:
                continue
            for wname, fused in inner.lora.items():
                w = getattr(inner, wname)
                for p in fused.parts:
                    w[p.row0:p.row0 + p.rows] += p.delta_weight().to(w.dtype)
            inner.lora = None
    for p in model.parameters():
        p.requires_grad_(True)
    return model


@reference_kwargs(config="lora_cfg")
def apply_lora(model, lora_cfg):
    """From a SOTAConfig `lora` section."""
    return get_peft_model(model, lora_cfg.r, lora_cfg.lora_alpha, lora_cfg.lora_dropout, list(lora_cfg.target_modules),
                          lora_cfg.use_rslora, list(lora_cfg.modules_to_save or []), lora_cfg.init_lora_weights,
                          dict(lora_cfg.rank_pattern or {}))


def lora_state_dict(model) -> dict[str, torch.Tensor]:
    return {n: p.detach().cpu() for n, p in model.named_parameters() if "lora_" in n}


def count_trainable(model) -> tuple[int, int]:
    t = sum(p.numel() for p in model.parameters() if p.requires_grad)
    return t, sum(p.numel() for p in model.parameters())


def _adapter_items(model):
    """(PEFT-style key stem, LoRALinear) for every adapter of the model, e.g.
    base_model.model.model.layers.3.self_attn.q_proj -> that layer's q adapter."""
    targets = _targets_for(model.config)
    by_slot = {(kind, w, row0): name for name, (kind, w, row0, _) in targets.items()}
    for li, layer in enumerate(model.model.layers):
        for kind, mod, hf in (("attn", layer.self_attn, "self_attn"), ("mlp", layer.mlp, "mlp")):
            inner = getattr(mod, "inner", mod)
            if getattr(inner, "lora", None) is None:
                continue
            for wname, fused in inner.lora.items():
                for p in fused.parts:
                    yield f"base_model.model.model.layers.{li}.{hf}.{by_slot[(kind, wname, p.row0)]}", p


def save_adapter(model, path, adapter_config: dict | None = None) -> None:
    """Writes `adapter_model.safetensors` (PEFT key layout: <module>.lora_A.weight / .lora_B.weight) and
    `adapter_config.json`, so that the adapter also loads with the peft package on a HuggingFace Llama."""
    import json
    from pathlib import Path
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    sd, ranks, targets, scale = {}, set(), set(), None
    for stem, p in _adapter_items(model):
        sd[f"{stem}.lora_A.weight"] = p.lora_A.detach().cpu().contiguous()
        sd[f"{stem}.lora_B.weight"] = p.lora_B.detach().cpu().contiguous()
        ranks.add(p.r)
        targets.add(stem.rsplit(".", 1)[1])
        scale = p.scaling
    try:
        from safetensors.torch import save_file
        save_file(sd, str(path / "adapter_model.safetensors"))
    except ImportError:
        torch.save(sd, path / "adapter_model.bin")
    r = max(ranks) if ranks else 0
    cfg = {"peft_type": "LORA", "r": r, "target_modules": sorted(targets), "scaling": scale,
           "lora_alpha": (scale or 0) * r, "use_rslora": False, "bias": "none", "task_type": "CAUSAL_LM"}
    cfg.update(adapter_config or {})
    (path / "adapter_config.json").write_text(json.dumps(cfg, indent=2))


def _read_adapter_file(path) -> dict[str, torch.Tensor]:
    from pathlib import Path
    path = Path(path)
    f = path / "adapter_model.safetensors"
    if f.exists():
        from safetensors.torch import load_file
        sd = load_file(str(f))
    else:
        sd = torch.load(path / "adapter_model.bin", map_location="cpu", weights_only=True)
    # peft inserts the adapter name ("default") before ".weight"
    return {k.replace(".lora_A.default.", ".lora_A.").replace(".lora_B.default.", ".lora_B."): v for k, v in sd.items()}


def adapter_state_from_dir(model, path) -> dict[str, torch.Tensor]:
    """An adapter directory (`save_adapter` / peft layout) as {parameter name of `model`: tensor}, the form of
    `lora_state_dict` that the serving engine's adapter registry takes; the model's own adapters are not touched."""
    sd = _read_adapter_file(path)
    names = {id(p): n for n, p in model.named_parameters()}
    out = {}
    for stem, part in _adapter_items(model):
        for kind in ("lora_A", "lora_B"):
            k = f"{stem}.{kind}.weight"
            if k not in sd:
                raise KeyError(f"adapter checkpoint has no {k}")
            out[names[id(getattr(part, kind))]] = sd[k]
    return out


def load_adapter(model, path, strict: bool = True) -> list[str]:
    """Loads adapter weights saved by `save_adapter` (or by peft, same key layout) into a model that already carries
    adapters of the same shapes (`get_peft_model` first).  Returns the keys that found no adapter."""
    sd = _read_adapter_file(path)
    used = set()
    with torch.no_grad():
        for stem, p in _adapter_items(model):
            for part, dst in (("lora_A", p.lora_A), ("lora_B", p.lora_B)):
                k = f"{stem}.{part}.weight"
                if k in sd:
                    dst.copy_(sd[k].to(dst.dtype))
                    used.add(k)
                elif strict:
                    raise KeyError(f"adapter checkpoint has no {k}")
    return sorted(set(sd) - used)


# ------------------------------------------------------------------------------------------------ names of the reference
@dataclass
class LoraConfig:
    """Adapter hyper-parameters (data_pipeline/trainer/lora.py:27-62); `apply_lora(model, LoraConfig(...))` applies
    them.  `scaling` = alpha / r, or alpha / sqrt(r) with rank-stabilised LoRA."""
    r: int = 16
    lora_alpha: float = 32
    lora_dropout: float = 0.0
    target_modules: list = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                          "up_proj", "down_proj"])
    modules_to_save: list = field(default_factory=lambda: ["embed_tokens", "lm_head"])
    bias: str = "none"
    use_rslora: bool = False
    use_dora: bool = False
    init_lora_weights: bool | str = True
    rank_pattern: dict = field(default_factory=dict)

    @property
    def scaling(self) -> float:
        return self.lora_alpha / math.sqrt(self.r) if self.use_rslora else self.lora_alpha / self.r


def get_trainable_parameters(model) -> tuple[int, int, float]:
    """(trainable, total, percentage)."""
    trainable, total = count_trainable(model)
    return trainable, total, (100.0 * trainable / total if total else 0.0)


def print_trainable_parameters(model) -> None:
    t, n, pct = get_trainable_parameters(model)
    print(f"trainable params: {t:,d} || all params: {n:,d} || trainable%: {pct:.4f}")


def get_lora_state_dict(model) -> dict[str, torch.Tensor]:
    """The adapter tensors alone, by parameter name (data_pipeline/trainer/lora.py:298-304)."""
    return {n: p.data for n, p in model.named_parameters() if "lora_" in n}


def load_lora_weights(model, lora_weights: dict) -> int:
    """Copy adapter tensors (as `get_lora_state_dict` returns them) into a model that already has the adapters;
    returns the number of tensors loaded.  Names the model does not have are ignored, shapes must match."""
    own = dict(model.named_parameters())
    n = 0
    with torch.no_grad():
        for name, w in lora_weights.items():
            if name in own:
                own[name].copy_(w.to(own[name].dtype))
                n += 1
    return n
