"""The reference's import paths, served by this package.

Code written against generalaimodels/TrainScale imports from `data_pipeline...`
(`from data_pipeline.trainer.kernels import flash_attention`, `from data_pipeline.pipeline import DataPipeline`).
After

    import trainscale_b200.reference_paths          # or: trainscale_b200.reference_paths.install()

those statements resolve to this package's objects of the same names, so a script can be pointed at this framework
without editing its imports.  Nothing is installed unless this module is imported, and a real `data_pipeline` package
on `sys.path` is never shadowed (`install()` then refuses, unless `force=True`).

How a name is found: the reference path selects which of our modules are searched first (`_ROUTES`: e.g. anything under
`data_pipeline.trainer.distributed.context_parallel` looks in `parallel.cp` first), then every module of the package
is searched.  Where the POSITIONAL conventions of a function differ between the two sides (`flash_attention`: the
reference passes [batch, heads, seq, dim] and is not causal by default), the name resolves to the variant with the
reference's conventions (the function's `__reference_form__`), so positional calls mean what they meant there.
`from data_pipeline.trainer import inference` style imports of whole sub-packages resolve to our
sub-package of that name.  Any dotted path below `data_pipeline` is importable; a name this package does not have
raises ImportError as usual.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import pkgutil
import sys
import types

ROOT = "data_pipeline"
_OURS = __name__.rsplit(".", 1)[0]

# reference path prefix (longest match wins) -> our modules searched first, in order
_ROUTES: dict[str, tuple[str, ...]] = {
    "core.types": ("core.types",),
    "core.errors": ("core.errors",),
    "core.config_schema": ("config.data_schema",),
    "core": ("core.types", "core.errors", "config.data_schema"),
    "pipeline": ("data.pipeline",),
    "preprocessing.tokenization": ("data.tokenization",),
    "preprocessing.prompt_engine": ("data.prompt_engine",),
    "preprocessing.length_manager": ("data.length_manager",),
    "preprocessing": ("data.tokenization", "data.prompt_engine", "data.length_manager"),
    "data.dataset_wrappers": ("data.dataset_wrappers",),
    "data.collate": ("data.collate",),
    "data.dataloader_factory": ("data.dataloader_factory",),
    "data": ("data.dataset_wrappers", "data.collate", "data.dataloader_factory", "data.packing", "data.pipeline"),
    "introspection": ("introspection",),
    "trainer.core.types": ("core.types",),
    "trainer.core.errors": ("core.errors",),
    "trainer.core.sota_config": ("config.sota_config",),
    "trainer.core.config": ("config.training_args", "config.sota_config"),
    "trainer.core": ("config.sota_config", "config.training_args", "core.types", "core.errors"),
    "trainer.training_config": ("config.training_args",),
    "trainer.trainers": ("trainer.sota_trainer", "trainer.base"),
    "trainer.base": ("trainer.base",),
    "trainer.kernels.flex_attention": ("kernels.flex", "kernels"),
    "trainer.kernels.moe_kernels": ("kernels.moe", "kernels"),
    "trainer.kernels.compiler": ("utils.cuda_graphs", "kernels.compat", "kernels"),
    "trainer.kernels.distributed_kernels": ("parallel.dist_kernels",),
    "trainer.kernels.benchmark_suite": ("benchmark_suite",),
    "trainer.kernels": ("kernels", "kernels.compat", "kernels.flex", "kernels.moe", "utils.cuda_graphs",
                        "parallel.dist_kernels", "benchmark_suite"),
    "trainer.distributed.ddp": ("parallel.ddp",),
    "trainer.distributed.fsdp2": ("parallel.fsdp2",),
    "trainer.distributed.tensor_parallel": ("parallel.tp",),
    "trainer.distributed.pipeline_parallel": ("parallel.pipeline",),
    "trainer.distributed.zbpp": ("parallel.zbpp",),
    "trainer.distributed.context_parallel": ("parallel.cp",),
    "trainer.distributed.hybrid_cp_scheduler": ("parallel.cp",),
    "trainer.distributed.expert_parallel": ("parallel.ep",),
    "trainer.distributed.activation_checkpoint": ("parallel.activation",),
    "trainer.distributed.activation_offload": ("parallel.activation", "parallel.dist_utils"),
    "trainer.distributed.grad_buffer": ("parallel.grad_buffer",),
    "trainer.distributed.parallel_dims": ("parallel.mesh",),
    "trainer.distributed.reduce_scatter_fp32": ("parallel.dist_utils",),
    "trainer.distributed": ("parallel.dist_utils", "parallel.ddp", "parallel.fsdp2", "parallel.tp", "parallel.pipeline",
                            "parallel.zbpp", "parallel.cp", "parallel.ep", "parallel.activation", "parallel.grad_buffer",
                            "parallel.mesh", "parallel.dist_kernels"),
    "trainer.loss": ("losses", "losses.extra"),
    "trainer.optimizers": ("optim",),
    "trainer.schedulers": ("schedulers",),
    "trainer.metrics": ("metrics", "metrics.trackers", "metrics.throughput"),
    "trainer.callbacks": ("callbacks",),
    "trainer.hub": ("hub",),
    "trainer.registry": ("registry", "registry.catalog", "core.types"),
    "trainer.lora": ("lora",),
    "trainer.quantization": ("quantization",),
    "trainer.export": ("export",),
    "trainer.rl": ("rl",),
    "trainer.rl_training": ("rl",),
    "trainer.inference": ("inference", "inference.engine"),
    "trainer": ("trainer.sota_trainer", "trainer.base", "config.sota_config", "config.training_args"),
}

_index: dict[str, object] | None = None


def _global_index() -> dict[str, object]:
    """name -> object over every module of this package; a name's defining module wins over modules that re-export it."""
    global _index
    if _index is not None:
        return _index
    pkg = importlib.import_module(_OURS)
    defined: dict[str, object] = {}
    seen: dict[str, object] = {}
    for m in pkgutil.walk_packages(pkg.__path__, _OURS + "."):
        if m.name.endswith("__main__") or m.name == __name__:
            continue
        try:
            mod = importlib.import_module(m.name)
        except Exception:   # noqa: BLE001 - optional dependencies of single modules
            continue
        for n, v in vars(mod).items():
            if n.startswith("_") or isinstance(v, types.ModuleType):
                continue
            seen.setdefault(n, v)
            if getattr(v, "__module__", None) == m.name:
                defined.setdefault(n, v)
    seen.update(defined)
    _index = seen
    return _index


def _routed_modules(ref_path: str) -> list[types.ModuleType]:
    rel = ref_path[len(ROOT):].lstrip(".")
    best = ""
    for prefix in _ROUTES:
        if (rel == prefix or rel.startswith(prefix + ".")) and len(prefix) > len(best):
            best = prefix
    out = []
    for name in _ROUTES.get(best, ()):
        try:
            out.append(importlib.import_module(f"{_OURS}.{name}"))
        except Exception:   # noqa: BLE001
            continue
    return out


class _ReferenceModule(types.ModuleType):
    """Stand-in for one module (or package) of the reference: attributes are looked up in this framework on demand."""

    def __getattr__(self, name: str):
        if name.startswith("__"):
            raise AttributeError(name)
        for mod in _routed_modules(self.__name__):
            if hasattr(mod, name):
                value = getattr(mod, name)
                break
        else:
            value = _global_index().get(name)
            if value is None:
                try:                                     # a whole sub-package: `from data_pipeline.trainer import inference`
                    value = importlib.import_module(f"{_OURS}.{name}")
                except ImportError:
                    raise AttributeError(f"{self.__name__}: {_OURS} has no counterpart of {name!r}") from None
        value = getattr(value, "__reference_form__", value)   # same op, the reference's positional order and layout
        setattr(self, name, value)
        return value


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname == ROOT or fullname.startswith(ROOT + "."):
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        mod = _ReferenceModule(spec.name)
        mod.__path__ = []                                # a package: any dotted path below it can be imported
        return mod

    def exec_module(self, module):
        module.__doc__ = f"Names of the reference's `{module.__name__}`, served by {_OURS}."


_finder: _Finder | None = None


def install(force: bool = False) -> bool:
    """Serve `data_pipeline...` imports from this package.  Returns True when the hook is (already) in place; refuses
    (False) when a real `data_pipeline` package is importable, unless `force`."""
    global _finder
    if _finder is not None:
        return True
    if not force:
        if ROOT in sys.modules and not isinstance(sys.modules[ROOT], _ReferenceModule):
            return False
        try:
            if importlib.util.find_spec(ROOT) is not None:
                return False
        except (ImportError, ValueError):
            pass
    _finder = _Finder()
    sys.meta_path.append(_finder)                        # last: never ahead of a real package
    if force:
        sys.meta_path.remove(_finder)
        sys.meta_path.insert(0, _finder)
        for k in [k for k in sys.modules if k == ROOT or k.startswith(ROOT + ".")]:
            del sys.modules[k]
    return True


def uninstall() -> None:
    global _finder
    if _finder is not None:
        sys.meta_path.remove(_finder)
        _finder = None
    for k in [k for k in sys.modules if (k == ROOT or k.startswith(ROOT + ".")) and isinstance(sys.modules[k], _ReferenceModule)]:
        del sys.modules[k]


install()
