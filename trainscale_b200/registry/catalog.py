"""Per-checkpoint model catalogue and the contract / capability helpers of the reference's registry.

`registry/__init__.py` describes model FAMILIES (what the framework decoder can load and how to patch them).  The
reference additionally keeps one record per published CHECKPOINT - organisation, base name, version, size, instruct
tag, quantisation flavour - keyed by its HuggingFace path, filled in by one `register_<family>_models()` function per
family (data_pipeline/trainer/registry/__init__.py:779-990 and the `_llama.py` ... `_vision_models.py` files).  This
module provides that catalogue from one compact table, plus the typed contract errors, `BaseModuleContract`, capability
decorators and the layer-patch table of the same file (:190-330, :758-772, :997-1000, :1180-1190).

Checkpoints in their original precision are listed under their publisher; pre-quantised variants (bitsandbytes, GGUF,
dynamic 4-bit) under the organisation that hosts them ("unsloth"), as in the reference.
"""
from __future__ import annotations

import functools
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Optional

import torch.nn as nn


class QuantType(Enum):
    NONE = "none"
    BNB_4BIT = "bnb-4bit"
    BNB_8BIT = "bnb-8bit"
    FP8 = "fp8"
    GGUF = "gguf"
    DYNAMIC = "dynamic"
    BF16 = "bf16"


QUANT_TAG_MAP = {QuantType.NONE: None, QuantType.BNB_4BIT: "bnb-4bit", QuantType.BNB_8BIT: "bnb-8bit",
                 QuantType.FP8: "fp8", QuantType.GGUF: "GGUF", QuantType.DYNAMIC: "unsloth-bnb-4bit",
                 QuantType.BF16: "bf16"}
QUANT_HOST_ORG = "unsloth"


@dataclass
class CheckpointInfo:
    """One published checkpoint.  `name` is derived from the parts unless given."""
    org: str
    base_name: str
    version: str
    size: str
    name: Optional[str] = None
    is_multimodal: bool = False
    instruct_tag: Optional[str] = None
    quant_type: QuantType = QuantType.NONE
    description: Optional[str] = None
    attention_class: Optional[str] = None
    mlp_class: Optional[str] = None
    layernorm_class: Optional[str] = None
    rope_class: Optional[str] = None

    def __post_init__(self):
        if self.name is None:
            self.name = self.construct_model_name(self.base_name, self.version, self.size, self.quant_type,
                                                  self.instruct_tag)

    @classmethod
    def construct_model_name(cls, base_name: str, version: str, size: str, quant_type: QuantType = QuantType.NONE,
                             instruct_tag: Optional[str] = None) -> str:
        parts = [base_name] + ([version] if version else []) + ([f"{size}B"] if size and size != "default" else [])
        if instruct_tag:
            parts.append(instruct_tag)
        tag = QUANT_TAG_MAP.get(quant_type)
        if tag:
            parts.append(tag)
        return "-".join(parts)

    @property
    def model_path(self) -> str:
        return f"{self.org}/{self.name}"


class LlamaModelInfo(CheckpointInfo): ...
class QwenModelInfo(CheckpointInfo): ...
class GemmaModelInfo(CheckpointInfo): ...
class MistralModelInfo(CheckpointInfo): ...
class DeepSeekModelInfo(CheckpointInfo): ...


@dataclass
class FamilyMeta:
    """A family release: the cross product sizes x instruct tags x quantisation flavours is what gets registered."""
    org: str
    base_name: str
    model_version: str
    model_info_cls: type = CheckpointInfo
    model_sizes: list = field(default_factory=list)
    instruct_tags: list = field(default_factory=lambda: [None])
    quant_types: list = field(default_factory=lambda: [QuantType.NONE])
    is_multimodal: bool = False
    attention_class: Optional[str] = None
    mlp_class: Optional[str] = None
    layernorm_class: Optional[str] = None
    rope_class: Optional[str] = None


CHECKPOINT_REGISTRY: dict[str, CheckpointInfo] = {}
LAYER_PATCHES: dict[str, Callable] = {}


def register_model(model_info_cls: type, org: str, base_name: str, version: str, size: str,
                   instruct_tag: Optional[str] = None, quant_type: QuantType = QuantType.NONE,
                   is_multimodal: bool = False, name: Optional[str] = None, **kwargs) -> Optional[CheckpointInfo]:
    """Add one checkpoint; a key that exists already is left alone (None is returned)."""
    info = model_info_cls(org=org, base_name=base_name, version=version, size=size, name=name,
                          is_multimodal=is_multimodal, instruct_tag=instruct_tag, quant_type=quant_type, **kwargs)
    if info.model_path in CHECKPOINT_REGISTRY:
        return None
    CHECKPOINT_REGISTRY[info.model_path] = info
    return info


def register_family(meta: FamilyMeta, include_original: bool = True) -> int:
    """Register every variant of a family release; returns how many were new."""
    n = 0
    layer = dict(attention_class=meta.attention_class, mlp_class=meta.mlp_class, layernorm_class=meta.layernorm_class,
                 rope_class=meta.rope_class)
    for size in meta.model_sizes:
        for tag in meta.instruct_tags:
            for q in meta.quant_types:
                if q is QuantType.NONE and not include_original:
                    continue
                org = meta.org if q is QuantType.NONE else QUANT_HOST_ORG
                n += register_model(meta.model_info_cls, org, meta.base_name, meta.model_version, size, tag, q,
                                    meta.is_multimodal, **layer) is not None
    return n


def search_models(base_name: Optional[str] = None, quant_type: Optional[QuantType] = None,
                  is_multimodal: Optional[bool] = None, org: Optional[str] = None) -> list[CheckpointInfo]:
    return [i for i in CHECKPOINT_REGISTRY.values()
            if (base_name is None or i.base_name == base_name) and (quant_type is None or i.quant_type == quant_type)
            and (is_multimodal is None or i.is_multimodal == is_multimodal) and (org is None or i.org == org)]


def get_checkpoint_info(model_id: str) -> Optional[CheckpointInfo]:
    return CHECKPOINT_REGISTRY.get(model_id)


# ------------------------------------------------------------------------------------------------ the table
_Q4 = [QuantType.NONE, QuantType.BNB_4BIT]
_QD = [QuantType.NONE, QuantType.BNB_4BIT, QuantType.DYNAMIC]
_QG = [QuantType.NONE, QuantType.BNB_4BIT, QuantType.DYNAMIC, QuantType.GGUF]


def _layers(prefix: str, norm: str = "RMSNorm", rope: bool = True) -> dict:
    return dict(attention_class=f"{prefix}Attention", mlp_class=f"{prefix}MLP", layernorm_class=f"{prefix}{norm}",
                rope_class=f"{prefix}RotaryEmbedding" if rope else None)


# family -> list of (org, base name, version, sizes, instruct tags, quant flavours, info class, multimodal, layer classes)
_FAMILIES: dict[str, list[tuple]] = {
    "llama": [
        ("meta-llama", "Llama", "3.1", ["8", "70", "405"], [None, "Instruct"], _QD, LlamaModelInfo, False, _layers("Llama")),
        ("meta-llama", "Llama", "3.2", ["1", "3"], [None, "Instruct"], _QG, LlamaModelInfo, False, _layers("Llama")),
        ("meta-llama", "Llama", "3.2", ["11", "90"], ["Vision", "Vision-Instruct"], _Q4, LlamaModelInfo, True, _layers("Llama")),
        ("meta-llama", "Llama", "3.3", ["70"], ["Instruct"], _QD, LlamaModelInfo, False, _layers("Llama")),
    ],
    "qwen": [
        ("Qwen", "Qwen", "2.5", ["0.5", "1.5", "3", "7", "14", "32", "72"], [None, "Instruct"], _QD, QwenModelInfo, False, _layers("Qwen2")),
        ("Qwen", "Qwen", "2.5-Coder", ["1.5", "7", "14", "32"], [None, "Instruct"], _Q4, QwenModelInfo, False, _layers("Qwen2")),
        ("Qwen", "QwQ", "", ["32"], ["Preview"], _Q4, QwenModelInfo, False, _layers("Qwen2")),
        ("Qwen", "Qwen", "2.5-VL", ["3", "7", "72"], ["Instruct"], _Q4, QwenModelInfo, True, _layers("Qwen2_5_VL")),
    ],
    "gemma": [
        ("google", "gemma", "2", ["2", "9", "27"], [None, "it"], _QD, GemmaModelInfo, False, _layers("Gemma2")),
        ("google", "gemma", "3", ["1", "4", "12", "27"], [None, "it"], _QD, GemmaModelInfo, False, _layers("Gemma3")),
    ],
    "mistral": [
        ("mistralai", "Mistral", "0.3", ["7"], [None, "Instruct"], _QD, MistralModelInfo, False, _layers("Mistral")),
        ("mistralai", "Mistral-Small", "24.09", ["22"], [None, "Instruct"], _Q4, MistralModelInfo, False, _layers("Mistral")),
        ("mistralai", "Mistral-Nemo", "24.07", ["12"], ["Base", "Instruct"], _Q4, MistralModelInfo, False, _layers("Mistral")),
    ],
    "deepseek": [
        ("deepseek-ai", "DeepSeek", "V3", ["default"], [None, "Chat"], [QuantType.NONE, QuantType.BF16, QuantType.FP8], DeepSeekModelInfo, False, _layers("DeepseekV3")),
        ("deepseek-ai", "DeepSeek", "R1", ["default", "7", "14", "32", "70"], [None, "Distill-Llama", "Distill-Qwen"], _QD, DeepSeekModelInfo, False, _layers("DeepseekV3")),
    ],
    "phi": [
        ("microsoft", "Phi-3", "3", ["3.8", "7", "14"], [None, "Instruct", "128k-Instruct", "4k-Instruct"], _Q4, CheckpointInfo, False, _layers("Phi3")),
        ("microsoft", "Phi-4", "4", ["14"], [None, "Instruct"], _QD, CheckpointInfo, False, _layers("Phi3")),
    ],
    "yi": [
        ("01-ai", "Yi", "1", ["6", "9", "34"], [None, "Chat", "200K"], _Q4, CheckpointInfo, False, _layers("Llama")),
        ("01-ai", "Yi-1.5", "1.5", ["6", "9", "34"], [None, "Chat", "Chat-16K"], _Q4, CheckpointInfo, False, _layers("Llama")),
        ("01-ai", "Yi-Coder", "1.5", ["1.5", "9"], [None, "Chat"], _Q4, CheckpointInfo, False, _layers("Llama")),
    ],
    "falcon": [
        ("tiiuae", "falcon", "1", ["7", "40", "180"], [None, "instruct"], _Q4, CheckpointInfo, False, _layers("Falcon", "LayerNorm")),
        ("tiiuae", "falcon2", "2", ["11"], [None, "instruct"], _Q4, CheckpointInfo, False, _layers("Falcon", "LayerNorm")),
        ("tiiuae", "Falcon-H1", "H1", ["0.5", "1.5", "3", "7", "34"], [None, "Instruct", "Deep-Instruct"], _Q4, CheckpointInfo, False, _layers("FalconH1")),
    ],
    "cohere_granite": [
        ("CohereForAI", "c4ai-command-r", "1", ["35", "104"], [None, "v01"], _Q4, CheckpointInfo, False, _layers("Cohere", "LayerNorm")),
        ("CohereForAI", "aya", "1", ["8", "35"], [None, "expanse"], _Q4, CheckpointInfo, False, _layers("Cohere", "LayerNorm")),
        ("ibm-granite", "granite", "3.0", ["1", "3", "8", "20"], [None, "instruct"], _Q4, CheckpointInfo, False, _layers("Granite")),
        ("ibm-granite", "granite-code", "3.0", ["3", "8", "20", "34"], [None, "instruct", "base"], _Q4, CheckpointInfo, False, _layers("Granite")),
    ],
    "code": [
        ("bigcode", "starcoder", "1", ["1", "3", "7", "15"], [None, "instruct"], [QuantType.NONE], CheckpointInfo, False, _layers("GPTBigCode", "LayerNorm", False)),
        ("bigcode", "starcoder2", "2", ["3", "7", "15"], [None, "instruct"], _Q4, CheckpointInfo, False, _layers("Starcoder2", "LayerNorm")),
        ("meta-llama", "CodeLlama", "1", ["7", "13", "34", "70"], [None, "Instruct", "Python"], _Q4, LlamaModelInfo, False, _layers("Llama")),
        ("deepseek-ai", "deepseek-coder", "1.3", ["1.3", "6.7", "33"], [None, "instruct", "base"], _Q4, DeepSeekModelInfo, False, _layers("Llama")),
        ("deepseek-ai", "DeepSeek-Coder-V2", "2", ["16", "236"], [None, "Instruct", "Lite-Instruct"], _Q4, DeepSeekModelInfo, False, _layers("DeepseekV2")),
        ("Qwen", "Qwen2.5-Coder", "2.5", ["0.5", "1.5", "3", "7", "14", "32"], [None, "Instruct"], _Q4, QwenModelInfo, False, _layers("Qwen2")),
    ],
    "moe": [
        ("mistralai", "Mixtral-8x7B", "0.1", ["8x7"], [None, "Instruct-v0.1"], _Q4, MistralModelInfo, False, dict(_layers("Mixtral"), mlp_class="MixtralSparseMoeBlock")),
        ("mistralai", "Mixtral-8x22B", "0.1", ["8x22"], [None, "Instruct-v0.1"], _Q4, MistralModelInfo, False, dict(_layers("Mixtral"), mlp_class="MixtralSparseMoeBlock")),
        ("Qwen", "Qwen1.5-MoE", "1.5", ["A2.7"], [None, "Chat"], _Q4, QwenModelInfo, False, dict(_layers("Qwen2Moe"), mlp_class="Qwen2MoeSparseMoeBlock")),
        ("Qwen", "Qwen3-MoE", "3", ["A3", "A22"], [None, "Instruct"], _Q4, QwenModelInfo, False, dict(_layers("Qwen3Moe"), mlp_class="Qwen3MoeSparseMoeBlock")),
        ("databricks", "dbrx", "1", ["132"], [None, "instruct"], _Q4, CheckpointInfo, False, dict(_layers("Dbrx", "LayerNorm"), mlp_class="DbrxFFN")),
        ("xai-org", "grok", "1", ["314"], [None], [QuantType.NONE], CheckpointInfo, False, dict(_layers("Grok1"), mlp_class="Grok1MoeBlock")),
    ],
    "vision": [
        ("llava-hf", "llava", "1.5", ["7", "13"], ["hf"], _Q4, CheckpointInfo, True, _layers("Llama")),
        ("llava-hf", "llava-v1.6", "1.6", ["7", "13", "34"], [None, "vicuna", "mistral"], _Q4, CheckpointInfo, True, _layers("Llama")),
        ("llava-hf", "llava-onevision", "0.5", ["0.5", "7", "72"], [None, "qwen2", "si"], _Q4, CheckpointInfo, True, _layers("Qwen2")),
        ("Qwen", "Qwen2-VL", "2", ["2", "7", "72"], [None, "Instruct"], _Q4, QwenModelInfo, True, _layers("Qwen2VL")),
        ("mistralai", "Pixtral", "24.09", ["12"], [None], _Q4, MistralModelInfo, True, _layers("Mistral")),
        ("OpenGVLab", "InternVL2", "2", ["1", "2", "8", "26", "40", "76"], [None, "Instruct"], _Q4, CheckpointInfo, True, _layers("InternLM2")),
    ],
}
_REGISTERED: set[str] = set()


def _family_meta(family: str, base_name: str, version: str | None = None, size: str | None = None) -> FamilyMeta:
    """The catalogue row of one release as a `FamilyMeta` (what `register_models_from_meta` / `register_family` take)."""
    for org, base, ver, sizes, tags, quants, cls, mm, layers in _FAMILIES[family]:
        if base == base_name and (version is None or ver == version) and (size is None or size in sizes):
            return FamilyMeta(org, base, ver, cls, list(sizes), list(tags), list(quants), mm, **layers)
    raise KeyError(f"no release {base_name!r} {version!r} in family {family!r}")


def _register(family: str, include_original: bool = True) -> int:
    if family in _REGISTERED:
        return 0
    _REGISTERED.add(family)
    n = 0
    for org, base, ver, sizes, tags, quants, cls, mm, layers in _FAMILIES[family]:
        n += register_family(FamilyMeta(org, base, ver, cls, sizes, tags, quants, mm, **layers), include_original)
    return n


def register_llama_models(include_original: bool = True) -> int: return _register("llama", include_original)
def register_qwen_models(include_original: bool = True) -> int: return _register("qwen", include_original)
def register_gemma_models(include_original: bool = True) -> int: return _register("gemma", include_original)
def register_mistral_models(include_original: bool = True) -> int: return _register("mistral", include_original)
def register_deepseek_models(include_original: bool = True) -> int: return _register("deepseek", include_original)
def register_phi_models(include_original: bool = True) -> int: return _register("phi", include_original)
def register_yi_models(include_original: bool = True) -> int: return _register("yi", include_original)
def register_falcon_models(include_original: bool = True) -> int: return _register("falcon", include_original)
def register_cohere_granite_models(include_original: bool = True) -> int: return _register("cohere_granite", include_original)
def register_code_models(include_original: bool = True) -> int: return _register("code", include_original)
def register_moe_models(include_original: bool = True) -> int: return _register("moe", include_original)
def register_vision_models(include_original: bool = True) -> int: return _register("vision", include_original)


def register_all_models(include_original: bool = True) -> int:
    return sum(_register(f, include_original) for f in _FAMILIES)


# ------------------------------------------------------------------------------------------------ contracts
@dataclass(frozen=True)
class ContractError:
    """Why a module contract could not be honoured (a value, not an exception: validation collects them)."""
    message: str
    module_name: str = ""


@dataclass(frozen=True)
class DependencyError(ContractError):
    missing_deps: tuple = ()
    cycle_path: tuple = ()


@dataclass(frozen=True)
class HardwareError(ContractError):
    required: tuple = ()
    available: tuple = ()


@dataclass(frozen=True)
class RegistrationError(ContractError):
    reason: str = ""


@dataclass
class BaseModuleContract:
    """A named, versioned kernel / patch with its dependencies, the hardware it needs and what to fall back to.
    `validate(hardware)` returns a list of `ContractError` values (empty = usable); `to_contract()` gives the compact
    form the capability matrix of `registry/__init__.py` stores."""
    _name: str
    _version: tuple = (1, 0, 0)
    _dependencies: frozenset = field(default_factory=frozenset)
    _hardware_requirements: frozenset = field(default_factory=frozenset)
    _fallback: Optional["BaseModuleContract"] = None
    _description: str = ""

    name = property(lambda self: self._name)
    version = property(lambda self: self._version)
    dependencies = property(lambda self: self._dependencies)
    hardware_requirements = property(lambda self: self._hardware_requirements)
    fallback = property(lambda self: self._fallback)
    description = property(lambda self: self._description)

    def validate(self, hardware=None, known: Optional[set] = None) -> list[ContractError]:
        from . import detect_capabilities
        hw = hardware if hardware is not None else detect_capabilities()
        errors: list[ContractError] = []
        lacking = tuple(c for c in self._hardware_requirements if not hw.has(c))
        if lacking:
            errors.append(HardwareError(f"{self._name} needs {[getattr(c, 'value', c) for c in lacking]}", self._name,
                                        required=tuple(self._hardware_requirements), available=tuple(hw.capabilities)))
        if known is not None:
            missing = tuple(sorted(d for d in self._dependencies if d not in known))
            if missing:
                errors.append(DependencyError(f"{self._name} depends on unregistered {list(missing)}", self._name,
                                              missing_deps=missing))
        return errors

    def get_fallback(self) -> Optional["BaseModuleContract"]:
        return self._fallback

    def version_string(self) -> str:
        return ".".join(str(v) for v in self._version)

    def to_contract(self):
        from . import ModuleContract
        return ModuleContract(self._name, tuple(self._hardware_requirements), tuple(sorted(self._dependencies)),
                              self._fallback.name if self._fallback is not None else None)


def has_capability(cap) -> bool:
    from . import detect_capabilities
    return detect_capabilities().has(cap)


def requires_capability(*caps) -> Callable:
    """Decorator: the function raises a RuntimeError naming the missing capabilities instead of failing inside a
    kernel launch."""
    def decorator(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            missing = [getattr(c, "name", str(c)) for c in caps if not has_capability(c)]
            if missing:
                raise RuntimeError(f"{fn.__name__} requires: {missing}")
            return fn(*args, **kwargs)
        return wrapper
    return decorator


_VALIDATOR = [None]


def get_registry_validator():
    """Process-wide `RegistryValidator` over the default capability matrix."""
    if _VALIDATOR[0] is None:
        from . import DEFAULT_CONTRACTS, KernelCapabilityMatrix, RegistryValidator
        _VALIDATOR[0] = RegistryValidator(KernelCapabilityMatrix(list(DEFAULT_CONTRACTS)))
    return _VALIDATOR[0]


# ------------------------------------------------------------------------------------------------ layer patches
def register_layer_patch(layer_class_name: str, patch_fn: Callable) -> None:
    """`patch_fn(module)` will be applied by `apply_layer_patches` to every module whose class has this name."""
    LAYER_PATCHES[layer_class_name] = patch_fn


def apply_layer_patches(model: nn.Module) -> list[str]:
    done = []
    for name, module in model.named_modules():
        fn = LAYER_PATCHES.get(type(module).__name__)
        if fn is not None and not getattr(module, "_ts_patched", False):
            fn(module)
            module._ts_patched = True
            done.append(name)
    return done


def _patch_gated_mlp(module: nn.Module, act: str) -> None:
    import types

    import torch

    from ..ops import activation as A
    from ..ops import gemm as G
    if not all(hasattr(module, k) for k in ("gate_proj", "up_proj", "down_proj")):
        return

    def fwd(self, x):
        gu = torch.cat((G.linear(x, self.gate_proj.weight, self.gate_proj.bias),
                        G.linear(x, self.up_proj.weight, self.up_proj.bias)), dim=-1)
        return G.linear(A.glu(gu, act), self.down_proj.weight, self.down_proj.bias)
    module.forward = types.MethodType(fwd, module)


def auto_patch_mlp_swiglu(module: nn.Module) -> None:
    _patch_gated_mlp(module, "silu")


def auto_patch_mlp_geglu(module: nn.Module) -> None:
    """Gemma-style MLP (GELU-tanh gate) of ONE module onto the framework GEMMs and the fused gate kernel."""
    _patch_gated_mlp(module, "gelu_tanh")


for _n in ("LlamaMLP", "Qwen2MLP", "Qwen3MLP", "MistralMLP", "Phi3MLP", "GraniteMLP"):
    register_layer_patch(_n, auto_patch_mlp_swiglu)
for _n in ("GemmaMLP", "Gemma2MLP", "Gemma3MLP"):
    register_layer_patch(_n, auto_patch_mlp_geglu)


# ---- one named constant per release, under the names of data_pipeline/trainer/registry/_*.py, built from the
# catalogue above (so that `register_models_from_meta(YI_15_META)` style code keeps working)
LlamaMeta_3_1 = _family_meta("llama", "Llama", "3.1")
LlamaMeta_3_2 = _family_meta("llama", "Llama", "3.2", "1")
LlamaMeta_3_2_Vision = LLAMA32_VISION_META = _family_meta("llama", "Llama", "3.2", "11")
QwenMeta_2_5 = _family_meta("qwen", "Qwen", "2.5")
QwenMeta_2_5_Coder = _family_meta("qwen", "Qwen", "2.5-Coder")
QwQMeta = _family_meta("qwen", "QwQ")
GemmaMeta_2 = _family_meta("gemma", "gemma", "2")
GemmaMeta_3 = _family_meta("gemma", "gemma", "3")
MistralMeta_7B = _family_meta("mistral", "Mistral", "0.3")
MistralMeta_Small = _family_meta("mistral", "Mistral-Small")
DeepSeekMeta_V3 = _family_meta("deepseek", "DeepSeek", "V3")
DeepSeekMeta_R1 = _family_meta("deepseek", "DeepSeek", "R1")
PHI_3_META = _family_meta("phi", "Phi-3")
PHI_4_META = _family_meta("phi", "Phi-4")
YI_1_META = _family_meta("yi", "Yi")
YI_15_META = _family_meta("yi", "Yi-1.5")
YI_CODER_META = _family_meta("yi", "Yi-Coder")
FALCON_1_META = _family_meta("falcon", "falcon")
FALCON_2_META = _family_meta("falcon", "falcon2")
FALCON_H1_META = _family_meta("falcon", "Falcon-H1")
COMMAND_R_META = _family_meta("cohere_granite", "c4ai-command-r")
AYA_META = _family_meta("cohere_granite", "aya")
GRANITE_META = _family_meta("cohere_granite", "granite")
GRANITE_CODE_META = _family_meta("cohere_granite", "granite-code")
STARCODER_META = _family_meta("code", "starcoder")
STARCODER2_META = _family_meta("code", "starcoder2")
CODELLAMA_META = _family_meta("code", "CodeLlama")
DEEPSEEK_CODER_META = _family_meta("code", "deepseek-coder")
DEEPSEEK_CODER_V2_META = _family_meta("code", "DeepSeek-Coder-V2")
QWEN_CODER_META = _family_meta("code", "Qwen2.5-Coder")
MIXTRAL_8x7B_META = _family_meta("moe", "Mixtral-8x7B")
MIXTRAL_8x22B_META = _family_meta("moe", "Mixtral-8x22B")
QWEN_MOE_META = _family_meta("moe", "Qwen1.5-MoE")
QWEN3_MOE_META = _family_meta("moe", "Qwen3-MoE")
DBRX_META = _family_meta("moe", "dbrx")
GROK_META = _family_meta("moe", "grok")
LLAVA_META = _family_meta("vision", "llava")
LLAVA_NEXT_META = _family_meta("vision", "llava-v1.6")
LLAVA_ONEVISION_META = _family_meta("vision", "llava-onevision")
QWEN_VL_META = _family_meta("vision", "Qwen2-VL")
QWEN25_VL_META = _family_meta("qwen", "Qwen", "2.5-VL")
PIXTRAL_META = _family_meta("vision", "Pixtral")
INTERNVL_META = _family_meta("vision", "InternVL2")
