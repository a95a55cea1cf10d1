"""Model-family registry, hardware capability probe, kernel capability matrix and the kernel patcher.

After data_pipeline/trainer/registry/__init__.py:57-1730 (`HardwareCapability`, `detect_capabilities`, `ModuleContract`,
`DependencyGraph` with Tarjan SCC + topological sort, `KernelCapabilityMatrix`, `RegistryValidator`, `ModelInfo`,
`register_models_from_meta`, `patch_model`, `KernelPatcher`) and the per-family tables `_llama.py` ... `_vision_models.py`.
The framework's own decoder is built on the sm_100a kernels, so "patching" here means converting a HuggingFace Llama-
family module tree into the framework decoder (`KernelPatcher.patch`), not monkey-patching forward methods.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Iterable

import torch
import torch.nn as nn

from ..utils.refargs import ANY, reference_kwargs


class Capability(str, Enum):
    BF16 = "bf16"
    FP8 = "fp8"
    TCGEN05 = "tcgen05"
    TMA = "tma"
    NVLINK_P2P = "nvlink_p2p"
    MULTICAST = "nvls_multicast"
    FLASH_ATTENTION = "flash_attention"
    FUSED_CE = "fused_cross_entropy"


@dataclass(frozen=True)
class HardwareCapability:
    device: str
    compute_capability: tuple[int, int]
    sm_count: int
    memory_gb: float
    capabilities: frozenset

    def has(self, c: Capability) -> bool:
        return c in self.capabilities


def detect_capabilities(device: int = 0) -> HardwareCapability:
    if not torch.cuda.is_available():
        return HardwareCapability("cpu", (0, 0), 0, 0.0, frozenset())
    p = torch.cuda.get_device_properties(device)
    cc = (p.major, p.minor)
    caps = set()
    if cc >= (8, 0):
        caps.add(Capability.BF16)
    if cc >= (8, 9):
        caps.add(Capability.FP8)
    if cc >= (9, 0):
        caps.add(Capability.TMA)
    if cc[0] == 10:
        caps |= {Capability.TCGEN05, Capability.FLASH_ATTENTION, Capability.FUSED_CE}
    if torch.cuda.device_count() > 1:
        try:
            if torch.cuda.can_device_access_peer(0, 1):
                caps.add(Capability.NVLINK_P2P)
        except Exception:   # noqa: BLE001
            pass
    return HardwareCapability(p.name, cc, p.multi_processor_count, p.total_memory / 2 ** 30, frozenset(caps))


@dataclass
class ModuleContract:
    """What a kernel-backed module needs and provides."""
    name: str
    requires: tuple[Capability, ...] = ()
    depends_on: tuple[str, ...] = ()
    fallback: str | None = None
    factory: Callable | None = None
    version: tuple = (1, 0, 0)

    def satisfied_by(self, hw: HardwareCapability) -> bool:
        return all(hw.has(c) for c in self.requires)

    # ---- the protocol of data_pipeline/trainer/registry/__init__.py:252-300
    @property
    def dependencies(self) -> frozenset:
        return frozenset(self.depends_on)

    @property
    def hardware_requirements(self) -> frozenset:
        return frozenset(self.requires)

    def validate(self, hardware: "HardwareCapability | None" = None):
        """Ok(None) when the device has every required capability, else Err(HardwareError) naming what is missing."""
        from ..core.types import Err, Ok
        from .catalog import HardwareError
        hw = hardware if hardware is not None else detect_capabilities()
        missing = tuple(c for c in self.requires if not hw.has(c))
        if missing:
            return Err(HardwareError(f"{self.name} needs {[c.value for c in missing]}", self.name, required=missing,
                                     available=tuple(hw.capabilities)))
        return Ok(None)

    def get_fallback(self) -> str | None:
        """NAME of the contract to use when this one's requirements are not met (the matrix resolves names)."""
        return self.fallback


class DependencyGraph:
    def __init__(self):
        self.edges: dict[str, set[str]] = {}
        self.declared: set[str] = set()       # nodes added themselves, as opposed to only named as a dependency

    @reference_kwargs(name="node", dependencies="deps")
    def add(self, node: str, deps: Iterable[str] = ()):
        deps = list(deps)
        self.declared.add(node)
        self.edges.setdefault(node, set()).update(deps)
        for d in deps:
            self.edges.setdefault(d, set())

    # ---- data_pipeline/trainer/registry/__init__.py:394-525
    add_module = add

    def remove_module(self, name: str) -> None:
        """Forget the module's own edges; it stays as a (now undeclared) node while others still depend on it."""
        self.declared.discard(name)
        if any(name in d for n, d in self.edges.items() if n != name):
            self.edges[name] = set()
        else:
            self.edges.pop(name, None)

    def get_dependencies(self, name: str) -> frozenset:
        return frozenset(self.edges.get(name, ()))

    def topological_sort(self):
        """Ok(order with every module after its dependencies) or Err(DependencyError with the first cycle)."""
        from ..core.types import Err, Ok
        from .catalog import DependencyError
        cycles = self.find_cycles()
        if cycles:
            return Err(DependencyError(f"circular dependencies: {sorted(cycles[0])}", cycle_path=tuple(sorted(cycles[0]))))
        return Ok(self.topological_order())

    def validate_dependencies(self, name: str):
        from ..core.types import Err, Ok
        from .catalog import DependencyError
        missing = tuple(sorted(d for d in self.edges.get(name, ()) if d not in self.declared))
        if missing:
            return Err(DependencyError(f"missing dependencies of {name!r}: {list(missing)}", name, missing_deps=missing))
        return Ok(None)

    def strongly_connected_components(self) -> list[list[str]]:
        """Tarjan's algorithm (iterative)."""
        index, low, on, stack, out, counter = {}, {}, set(), [], [], [0]
        for root in self.edges:
            if root in index:
                continue
            work = [(root, iter(sorted(self.edges[root])))]
            index[root] = low[root] = counter[0]
            counter[0] += 1
            stack.append(root)
            on.add(root)
            while work:
                v, it = work[-1]
                advanced = False
                for w in it:
                    if w not in index:
                        index[w] = low[w] = counter[0]
                        counter[0] += 1
                        stack.append(w)
                        on.add(w)
                        work.append((w, iter(sorted(self.edges[w]))))
                        advanced = True
                        break
                    if w in on:
                        low[v] = min(low[v], index[w])
                if advanced:
                    continue
                work.pop()
                if work:
                    low[work[-1][0]] = min(low[work[-1][0]], low[v])
                if low[v] == index[v]:
                    comp = []
                    while True:
                        w = stack.pop()
                        on.discard(w)
                        comp.append(w)
                        if w == v:
                            break
                    out.append(comp)
        return out

    def find_cycles(self) -> list[list[str]]:
        return [c for c in self.strongly_connected_components() if len(c) > 1 or c[0] in self.edges[c[0]]]

    def topological_order(self) -> list[str]:
        if self.find_cycles():
            raise ValueError(f"dependency cycle: {self.find_cycles()[0]}")
        seen, order = set(), []

        def visit(n):
            if n in seen:
                return
            seen.add(n)
            for d in sorted(self.edges[n]):
                visit(d)
            order.append(n)

        for n in sorted(self.edges):
            visit(n)
        return order


class KernelCapabilityMatrix:
    """Which contracts are usable on a device, with fallback chains."""

    def __init__(self, contracts: Iterable[ModuleContract] = ()):
        self.contracts = {c.name: c for c in contracts}

    def register(self, c: ModuleContract):
        self.contracts[c.name] = c

    def resolve(self, name: str, hw: HardwareCapability) -> str | None:
        seen = set()
        while name and name not in seen:
            seen.add(name)
            c = self.contracts.get(name)
            if c is None:
                return None
            if c.satisfied_by(hw):
                return name
            name = c.fallback
        return None

    def available(self, hw: HardwareCapability) -> dict[str, bool]:
        return {n: c.satisfied_by(hw) for n, c in self.contracts.items()}

    # ---- data_pipeline/trainer/registry/__init__.py:541-610
    def register_kernel(self, contract, fallback_chain: list[str] | None = None):
        """Ok(None), or Err(RegistrationError) when the name is taken.  `contract`: a ModuleContract or a
        catalog.BaseModuleContract; `fallback_chain`: names tried in order when its requirements are not met."""
        from ..core.types import Err, Ok
        from .catalog import RegistrationError
        c = contract.to_contract() if hasattr(contract, "to_contract") else contract
        if c.name in self.contracts:
            return Err(RegistrationError(f"kernel {c.name!r} already registered", c.name, reason="duplicate_registration"))
        self.contracts[c.name] = c
        if fallback_chain:
            self.__dict__.setdefault("chains", {})[c.name] = list(fallback_chain)
        return Ok(None)

    def get_optimal_kernel(self, kernel_name: str, hw: HardwareCapability | None = None) -> "ModuleContract | None":
        """The first usable contract among the named one, its explicit fallback chain, and its `fallback` links."""
        hw = hw if hw is not None else detect_capabilities()
        for name in [kernel_name] + self.__dict__.get("chains", {}).get(kernel_name, []):
            c = self.contracts.get(name)
            if c is not None and c.satisfied_by(hw):
                return c
        got = self.resolve(kernel_name, hw)
        return self.contracts[got] if got else None

    def get_all_kernels(self) -> dict:
        return dict(self.contracts)

    def get_available_kernels(self, hw: HardwareCapability | None = None) -> list[str]:
        hw = hw if hw is not None else detect_capabilities()
        return [n for n, c in self.contracts.items() if c.satisfied_by(hw)]


DEFAULT_CONTRACTS = [
    ModuleContract("gemm_tcgen05", (Capability.TCGEN05, Capability.TMA), fallback="gemm_torch"),
    ModuleContract("gemm_torch"),
    ModuleContract("flash_attention_tcgen05", (Capability.TCGEN05,), ("gemm_tcgen05",), "attention_torch"),
    ModuleContract("attention_torch"),
    ModuleContract("rmsnorm_cuda", (Capability.BF16,), fallback="rmsnorm_torch"), ModuleContract("rmsnorm_torch"),
    ModuleContract("fused_linear_ce", (Capability.TCGEN05,), ("gemm_tcgen05",), "ce_torch"), ModuleContract("ce_torch"),
    ModuleContract("fused_collectives", (Capability.NVLINK_P2P,), ("gemm_tcgen05",), "nccl"), ModuleContract("nccl"),
]


class RegistryValidator:
    def __init__(self, matrix: KernelCapabilityMatrix | None = None, hardware: HardwareCapability | None = None):
        self.matrix = matrix if matrix is not None else KernelCapabilityMatrix()
        self.hardware = hardware                      # None: probed when needed
        self.graph = DependencyGraph()
        for c in self.matrix.contracts.values():
            self.graph.add(c.name, c.depends_on)

    def _hw(self) -> HardwareCapability:
        return self.hardware if self.hardware is not None else detect_capabilities()

    # ---- incremental registration (data_pipeline/trainer/registry/__init__.py:630-775)
    def validate_contract(self, contract):
        """Hardware first, then that every dependency is registered, then that no cycle would appear."""
        from ..core.types import Err, Ok
        from .catalog import DependencyError
        c = contract.to_contract() if hasattr(contract, "to_contract") else contract
        r = c.validate(self._hw())
        if r.is_err():
            return r
        missing = tuple(sorted(d for d in c.depends_on if d not in self.matrix.contracts))
        if missing:
            return Err(DependencyError(f"missing dependencies: {list(missing)}", c.name, missing_deps=missing))
        before = {n: set(d) for n, d in self.graph.edges.items()}, set(self.graph.declared)
        self.graph.add(c.name, c.depends_on)
        cycles = self.graph.find_cycles()
        self.graph.edges, self.graph.declared = before
        if cycles:
            return Err(DependencyError(f"would introduce a circular dependency: {sorted(cycles[0])}", c.name,
                                       cycle_path=tuple(sorted(cycles[0]))))
        return Ok(None)

    def register(self, contract, *, skip_validation: bool = False):
        from ..core.types import Ok
        c = contract.to_contract() if hasattr(contract, "to_contract") else contract
        if not skip_validation:
            r = self.validate_contract(c)
            if r.is_err():
                return r
        r = self.matrix.register_kernel(c)
        if r.is_err():
            return r
        self.graph.add(c.name, c.depends_on)
        return Ok(None)

    def get_registration_order(self):
        return self.graph.topological_sort()

    def validate_all(self) -> dict:
        hw = self._hw()
        return {n: c.validate(hw) for n, c in self.matrix.contracts.items()}

    def get_capabilities_report(self) -> dict:
        hw, results = self._hw(), self.validate_all()
        return {"hardware_capabilities": sorted(getattr(c, "value", str(c)) for c in hw.capabilities),
                "available_kernels": self.matrix.get_available_kernels(hw), "total_registered": len(results),
                "validation_passed": sum(r.is_ok() for r in results.values()),
                "validation_failed": sum(r.is_err() for r in results.values())}

    def validate(self) -> list[str]:
        problems = []
        g = DependencyGraph()
        for c in self.matrix.contracts.values():
            g.add(c.name, c.depends_on)
            for d in c.depends_on:
                if d not in self.matrix.contracts:
                    problems.append(f"{c.name} depends on unknown contract {d}")
            if c.fallback and c.fallback not in self.matrix.contracts:
                problems.append(f"{c.name} falls back to unknown contract {c.fallback}")
        for cyc in g.find_cycles():
            problems.append(f"dependency cycle: {sorted(cyc)}")
        return problems


@dataclass
class ModelInfo:
    family: str
    org: str
    sizes: tuple[str, ...]
    architecture: str = "LlamaForCausalLM"
    attention: str = "gqa"
    mlp: str = "swiglu"
    norm: str = "rmsnorm"
    rope: str = "default"
    supported: bool = True          # convertible to the framework decoder
    notes: str = ""

    @classmethod
    def construct_model_name(cls, base_name: str, version: str, size: str, quant_type=None,
                             instruct_tag: str | None = None) -> str:
        """Checkpoint name from its parts, e.g. ("Llama", "3.1", "8", instruct_tag="Instruct") -> Llama-3.1-8B-Instruct
        (the rule of `catalog.CheckpointInfo`, data_pipeline/trainer/registry/__init__.py:841-858)."""
        from .catalog import CheckpointInfo, QuantType
        return CheckpointInfo.construct_model_name(base_name, version, size, quant_type or QuantType.NONE, instruct_tag)

    @property
    def model_path(self) -> str:
        """Hub prefix of the family: "<org>/<family>"; single checkpoints are `catalog.CheckpointInfo.model_path`."""
        return f"{self.org}/{self.family}"


MODEL_REGISTRY: dict[str, ModelInfo] = {}


@reference_kwargs(model_meta="meta")
def register_models_from_meta(meta, include_original: bool = True) -> int:
    """Family-level records (an iterable of `ModelInfo`) go to MODEL_REGISTRY; a `catalog.FamilyMeta` (one release: sizes x
    instruct tags x quantisation flavours, the reference's ModelMeta) registers its checkpoints in
    `catalog.CHECKPOINT_REGISTRY`.  Returns how many entries were added."""
    from .catalog import FamilyMeta, register_family
    if isinstance(meta, FamilyMeta):
        return register_family(meta, include_original)
    n = 0
    for m in meta:
        MODEL_REGISTRY[m.family] = m
        n += 1
    return n


register_models_from_meta([
    ModelInfo("llama", "meta-llama", ("1B", "3B", "8B", "70B", "405B"), rope="llama3"),
    ModelInfo("mistral", "mistralai", ("7B", "12B", "24B"), "MistralForCausalLM", notes="sliding window attention"),
    ModelInfo("qwen", "Qwen", ("0.5B", "1.5B", "7B", "14B", "32B", "72B"), "Qwen2ForCausalLM", notes="qkv bias"),
    ModelInfo("gemma", "google", ("2B", "7B", "9B", "27B"), "GemmaForCausalLM", mlp="geglu", notes="norm weight offset 1, logit soft-cap"),
    ModelInfo("phi", "microsoft", ("3.8B", "14B"), "Phi3ForCausalLM", notes="fused qkv / gate_up in the checkpoint"),
    ModelInfo("deepseek", "deepseek-ai", ("7B", "67B", "V2", "V3"), "DeepseekV3ForCausalLM", attention="mla", mlp="moe", supported=False),
    ModelInfo("falcon", "tiiuae", ("7B", "40B"), "FalconForCausalLM", attention="mqa", norm="layernorm", supported=False),
    ModelInfo("yi", "01-ai", ("6B", "9B", "34B")),
    ModelInfo("cohere", "CohereForAI", ("8B", "35B"), "CohereForCausalLM", norm="layernorm", supported=False),
    ModelInfo("granite", "ibm-granite", ("2B", "8B"), "GraniteForCausalLM"),
    ModelInfo("codellama", "codellama", ("7B", "13B", "34B")), ModelInfo("starcoder2", "bigcode", ("3B", "7B", "15B"), "Starcoder2ForCausalLM", mlp="gelu", norm="layernorm", supported=False),
    ModelInfo("mixtral", "mistralai", ("8x7B", "8x22B"), "MixtralForCausalLM", mlp="moe"),
    ModelInfo("qwen_moe", "Qwen", ("A2.7B", "A14B"), "Qwen2MoeForCausalLM", mlp="moe", supported=False,
              notes="shared expert + per-layer dense/sparse mix not covered"),
    ModelInfo("llava", "llava-hf", ("7B", "13B"), "LlavaForConditionalGeneration", supported=False, notes="vision tower not covered"),
])


@reference_kwargs(model_id="name_or_path")
def get_model_info(name_or_path: str) -> ModelInfo | None:
    n = name_or_path.lower()
    for fam, info in MODEL_REGISTRY.items():
        if fam in n or info.org.lower() in n:
            return info
    return None


def convert_hf_llama(hf_model, dtype=torch.bfloat16, device=None):
    """HuggingFace Llama-family module -> framework decoder with the same weights."""
    from ..models.llama import LlamaConfig, build_model
    c = hf_model.config
    cfg = LlamaConfig(vocab_size=c.vocab_size, hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
                      num_hidden_layers=c.num_hidden_layers, num_attention_heads=c.num_attention_heads,
                      num_key_value_heads=getattr(c, "num_key_value_heads", c.num_attention_heads),
                      head_dim=getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads,
                      rms_norm_eps=c.rms_norm_eps, rope_theta=getattr(c, "rope_theta", None) or
                      (getattr(c, "rope_parameters", None) or {}).get("rope_theta", 10000.0),
                      max_position_embeddings=c.max_position_embeddings,
                      tie_word_embeddings=bool(getattr(c, "tie_word_embeddings", False)),
                      sliding_window=getattr(c, "sliding_window", None) if getattr(c, "use_sliding_window", True) else None,
                      # Qwen2 has q / k / v biases without a config flag; Llama-style configs say so explicitly
                      attention_bias=any(k.endswith("q_proj.bias") for k in hf_model.state_dict()),
                      num_local_experts=int(getattr(c, "num_local_experts", 0) or 0),
                      num_experts_per_tok=int(getattr(c, "num_experts_per_tok", 2) or 2),
                      router_aux_loss_coef=float(getattr(c, "router_aux_loss_coef", 0.0) or 0.0)
                      if getattr(c, "output_router_logits", False) else 0.0,
                      model_type=getattr(c, "model_type", "llama"),
                      hidden_act={"gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_tanh"}.get(
                          getattr(c, "hidden_activation", None) or getattr(c, "hidden_act", "silu"),
                          getattr(c, "hidden_act", "silu")),
                      norm_weight_offset=1.0 if getattr(c, "model_type", "") == "gemma" else 0.0,
                      scale_embeddings=getattr(c, "model_type", "") == "gemma")
    if any(k.endswith("o_proj.bias") for k in hf_model.state_dict()):
        raise ValueError("output-projection biases are not supported by the framework decoder")
    m = build_model(cfg, dtype=dtype, device=device)
    m.load_hf_state_dict({k: v for k, v in hf_model.state_dict().items()}, strict=not cfg.tie_word_embeddings)
    return m


class KernelPatcher:
    def __init__(self, matrix: KernelCapabilityMatrix | None = None):
        self.matrix = matrix or KernelCapabilityMatrix(DEFAULT_CONTRACTS)
        self.hw = detect_capabilities()

    def plan(self) -> dict[str, str | None]:
        return {n: self.matrix.resolve(n, self.hw) for n in ("gemm_tcgen05", "flash_attention_tcgen05", "rmsnorm_cuda",
                                                              "fused_linear_ce", "fused_collectives")}

    def patch(self, model, dtype=torch.bfloat16, device=None, *, model_info=None):
        """Framework decoders pass through; HF Llama-family models are converted; anything else is returned as is.
        `model_info` (a `ModelInfo`, also accepted in `dtype`'s place as in the reference's `patch(model, model_info)`)
        names the architecture when the class name does not."""
        from ..models.llama import LlamaForCausalLM
        if dtype is not None and not isinstance(dtype, torch.dtype):
            model_info, dtype = dtype, torch.bfloat16
        if isinstance(model, LlamaForCausalLM):
            return model
        arch = type(model).__name__
        if model_info is not None and arch not in ("LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM",
                                                   "MixtralForCausalLM", "GemmaForCausalLM"):
            family = str(getattr(model_info, "architecture", None) or getattr(model_info, "model_type", "") or "").lower()
            arch = {"llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM", "qwen2": "Qwen2ForCausalLM",
                    "mixtral": "MixtralForCausalLM", "gemma": "GemmaForCausalLM"}.get(family, arch)
        if arch in ("LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM", "MixtralForCausalLM",
                    "GemmaForCausalLM") and \
                not any(k.endswith("o_proj.bias") for k in model.state_dict()):
            return convert_hf_llama(model, dtype, device)
        return model


def _patch_stats(model) -> dict:
    """How many norm / MLP / attention / rotary modules of `model` run on the framework's ops, and how many there are.
    The framework decoder counts as patched throughout; for other models a module counts once an `auto_patch_*`
    function has rewired it (data_pipeline/trainer/registry/__init__.py:1420-1450)."""
    from ..models.llama import LlamaForCausalLM
    native = isinstance(model, LlamaForCausalLM)
    stats = {f"{k}_{w}": 0 for k in ("layernorm", "mlp", "attention", "rope") for w in ("patched", "total")}
    for _, m in model.named_modules():
        cls = type(m).__name__
        kind = ("layernorm" if cls.endswith(("RMSNorm", "LayerNorm")) else "mlp" if cls.endswith(("MLP", "MoE")) else
                "attention" if cls.endswith("Attention") else "rope" if cls.endswith("RotaryEmbedding") else None)
        if kind is None:
            continue
        stats[f"{kind}_total"] += 1
        stats[f"{kind}_patched"] += bool(native or getattr(m, "_ts_patched", False))
    return stats


KernelPatcher.get_stats = lambda self, model: _patch_stats(model)


def patch_model(model, **kw):
    return KernelPatcher().patch(model, **kw)


# ------------------------------------------------------------------------------------------------ module-level patchers
# For models that are NOT converted to the framework decoder (other architectures, custom heads): swap the forward of
# recognisable sub-modules for the framework ops.  Weights and state-dict keys stay as they are.  Each patcher returns
# the number of modules it changed (data_pipeline/trainer/registry/__init__.py:1033-1300 has the same entry points).
def _is_rmsnorm(m: nn.Module) -> bool:
    return type(m).__name__.endswith("RMSNorm") and hasattr(m, "weight") and m.weight is not None and m.weight.dim() == 1


@reference_kwargs(module="model")
def auto_patch_layernorm(model: nn.Module) -> int:
    """`nn.LayerNorm` and `*RMSNorm` modules -> `ops.norm.layernorm` / `ops.norm.rmsnorm` (sm_100a kernels for bf16 CUDA
    rows, PyTorch maths otherwise)."""
    import types
    from ..ops import norm as N
    n = 0
    for m in model.modules():
        if getattr(m, "_ts_patched", False):
            continue
        if isinstance(m, nn.LayerNorm) and len(m.normalized_shape) == 1 and m.weight is not None:
            m.forward = types.MethodType(lambda self, x: N.layernorm(x, self.weight, self.bias, self.eps), m)
        elif _is_rmsnorm(m):
            eps = float(getattr(m, "variance_epsilon", getattr(m, "eps", 1e-6)) or 1e-6)
            off = 1.0 if "Gemma" in type(m).__name__ else 0.0       # Gemma stores w - 1
            m.forward = types.MethodType(
                lambda self, x, _e=eps, _o=off: N.rmsnorm(x, self.weight, _e, None, _o)[0], m)
        else:
            continue
        m._ts_patched = True
        n += 1
    return n


@reference_kwargs(module="model")
def auto_patch_mlp(model: nn.Module) -> int:
    """Gated MLPs (`gate_proj` / `up_proj` / `down_proj` without biases, SiLU or GELU gate) -> framework GEMMs and the
    fused gate * up kernel."""
    import types
    from ..ops import activation as A
    from ..ops import gemm as G
    n = 0
    for m in model.modules():
        if getattr(m, "_ts_patched", False):
            continue
        g, u, d = (getattr(m, k, None) for k in ("gate_proj", "up_proj", "down_proj"))
        if not all(isinstance(t, nn.Linear) and t.bias is None for t in (g, u, d)):
            continue
        act_name = type(getattr(m, "act_fn", nn.SiLU())).__name__.lower()
        kind = "silu" if "silu" in act_name or "swish" in act_name else "gelu_tanh" if "gelu" in act_name else None
        if kind is None:
            continue

        def fwd(self, x, _k=kind):
            gu = torch.cat((G.linear(x, self.gate_proj.weight), G.linear(x, self.up_proj.weight)), dim=-1)
            return G.linear(A.glu(gu, _k), self.down_proj.weight)
        m.forward = types.MethodType(fwd, m)
        m._ts_patched = True
        n += 1
    return n


@reference_kwargs(module="model")
def auto_patch_rope(model: nn.Module) -> int:
    """Replaces `apply_rotary_pos_emb` in the Python module that defines the model's attention class with a version on
    the framework rotary kernel (rotate-half layout, cos / sin of shape [B, S, D] as transformers passes them).
    Returns the number of patched modules (0 when the model's source has no such function)."""
    import sys
    from ..ops import rope as R
    seen, n = set(), 0
    for m in model.modules():
        mod = sys.modules.get(type(m).__module__)
        if mod is None or mod.__name__ in seen or not hasattr(mod, "apply_rotary_pos_emb"):
            continue
        seen.add(mod.__name__)
        if getattr(mod.apply_rotary_pos_emb, "_ts_patched", False):
            continue
        orig = mod.apply_rotary_pos_emb

        def patched(q, k, cos, sin, position_ids=None, unsqueeze_dim=1, _orig=orig):
            # q, k: [B, H, S, D]; tables [B, S, D] with the two halves equal
            ok = q.dim() == 4 and cos.dim() == 3 and unsqueeze_dim == 1 and cos.shape[0] == 1 and q.is_cuda \
                and q.dtype == torch.bfloat16
            if not ok:
                return _orig(q, k, cos, sin, position_ids, unsqueeze_dim) if position_ids is not None \
                    else _orig(q, k, cos, sin, unsqueeze_dim=unsqueeze_dim)
            D = q.shape[-1]
            c, s = cos[0, :, : D // 2].float().contiguous(), sin[0, :, : D // 2].float().contiguous()
            qo = R.apply_rope(q.transpose(1, 2).contiguous(), c, s).transpose(1, 2)
            ko = R.apply_rope(k.transpose(1, 2).contiguous(), c, s).transpose(1, 2)
            return qo, ko
        patched._ts_patched = True
        mod.apply_rotary_pos_emb = patched
        n += 1
    return n


@reference_kwargs(module="model")
def auto_patch_fp8_linear(model: nn.Module, min_features: int = 1024, skip: tuple[str, ...] = ("lm_head",)) -> int:
    """Bias-free `nn.Linear` layers with both dimensions >= `min_features` and divisible by 128 -> block-scaled fp8
    GEMM (bf16 CUDA inputs; other inputs take the original path)."""
    import types
    from ..ops import fp8 as F8
    n = 0
    for name, m in model.named_modules():
        if not isinstance(m, nn.Linear) or m.bias is not None or getattr(m, "_ts_patched", False):
            continue
        if any(s in name for s in skip) or min(m.in_features, m.out_features) < min_features or \
                m.in_features % 128 or m.out_features % 128:
            continue

        def fwd(self, x):
            if F8.available(x) and self.weight.dtype == torch.bfloat16:
                return F8.fp8_linear(x, self.weight)
            return nn.functional.linear(x, self.weight)
        m.forward = types.MethodType(fwd, m)
        m._ts_patched = True
        n += 1
    return n


def auto_patch(model: nn.Module, layernorm: bool = True, mlp: bool = True, rope: bool = True, fp8: bool = False) -> dict:
    return {"layernorm": auto_patch_layernorm(model) if layernorm else 0, "mlp": auto_patch_mlp(model) if mlp else 0,
            "rope": auto_patch_rope(model) if rope else 0, "fp8_linear": auto_patch_fp8_linear(model) if fp8 else 0}


ModelMeta = ModelInfo          # name used by the per-family registration files of the reference


@reference_kwargs(module="model")
def auto_patch_attention(model: nn.Module, name: str = "trainscale_flash") -> int:
    """Registers the framework's flash attention with transformers' attention interface and switches the model's
    config to it, so that an unconverted HuggingFace model runs its attention on the tcgen05 kernels.  Calls that carry
    an explicit mask (padding), dropout, or non-bf16 / CPU tensors are handed to transformers' SDPA path.
    Returns the number of attention modules affected (0 when transformers has no such interface)."""
    try:
        from transformers import AttentionInterface
        from transformers.integrations.sdpa_attention import sdpa_attention_forward
    except Exception:
        return 0
    from ..kernels import flash_attention

    def forward(module, query, key, value, attention_mask, dropout: float = 0.0, scaling=None, is_causal=None, **kw):
        causal = is_causal if is_causal is not None else getattr(module, "is_causal", True)
        usable = attention_mask is None and not dropout and query.is_cuda and query.dtype == torch.bfloat16 \
            and query.shape[2] == key.shape[2] and query.shape[-1] in (64, 128) and not kw.get("sliding_window")
        if not usable:
            return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling,
                                          is_causal=is_causal, **kw)
        out = flash_attention(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), bool(causal), scaling)
        return out, None                                  # [B, S, H, D], as the interface expects

    AttentionInterface.register(name, forward)
    cfg = getattr(model, "config", None)
    if cfg is not None:
        cfg._attn_implementation = name
    n = 0
    for m in model.modules():
        if type(m).__name__.endswith("Attention") and hasattr(m, "config"):
            m.config._attn_implementation = name
            n += 1
    return n


# ------------------------------------------------------------------------------------------------ checkpoint catalogue
from .catalog import (CHECKPOINT_REGISTRY, LAYER_PATCHES, QUANT_TAG_MAP, BaseModuleContract, CheckpointInfo,  # noqa: E402,F401
                      ContractError, DeepSeekModelInfo, DependencyError, FamilyMeta, GemmaModelInfo, HardwareError,
                      LlamaModelInfo, MistralModelInfo, QuantType, QwenModelInfo, RegistrationError,
                      apply_layer_patches, auto_patch_mlp_geglu, auto_patch_mlp_swiglu, get_checkpoint_info,
                      get_registry_validator, has_capability, register_all_models, register_code_models,
                      register_cohere_granite_models, register_deepseek_models, register_falcon_models,
                      register_family, register_gemma_models, register_layer_patch, register_llama_models,
                      register_mistral_models, register_model, register_moe_models, register_phi_models,
                      register_qwen_models, register_vision_models, register_yi_models, requires_capability,
                      search_models)
