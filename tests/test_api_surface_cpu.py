"""Every public class / function name of the reference's package has a counterpart of the same name somewhere in this
package (a class, a function or a module-level alias).  The reference is read as text (its installed copy for the
comparison arm of bench.py, or a checkout named by TRAINSCALE_REFERENCE); the test is skipped where neither exists."""
import ast
import os
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _reference_root():
    for cand in (ROOT / "baseline" / "_ref" / "data_pipeline",
                 Path(os.environ.get("TRAINSCALE_REFERENCE", "/nonexistent")) / "data_pipeline"):
        if cand.is_dir():
            return cand
    return None


def _public_defs(root: Path) -> dict[str, str]:
    out = {}
    for p in root.rglob("*.py"):
        if "examples" in p.parts:
            continue
        try:
            tree = ast.parse(p.read_text())
        except SyntaxError:
            continue
        for node in tree.body:
            if isinstance(node, (ast.ClassDef, ast.FunctionDef)) and not node.name.startswith("_"):
                out.setdefault(node.name, str(p.relative_to(root)))
    return out


def _our_names(root: Path) -> set[str]:
    """Module-level classes, functions, assigned names and imported names of every file of the package."""
    names: set[str] = set()
    for p in root.rglob("*.py"):
        try:
            tree = ast.parse(p.read_text())
        except SyntaxError:
            continue
        for node in tree.body:
            if isinstance(node, (ast.ClassDef, ast.FunctionDef)):
                names.add(node.name)
            elif isinstance(node, (ast.Assign, ast.AnnAssign)):
                targets = node.targets if isinstance(node, ast.Assign) else [node.target]
                for t in targets:
                    for n in ast.walk(t):
                        if isinstance(n, ast.Name):
                            names.add(n.id)
    return names


def test_every_public_name_of_the_reference_exists_here():
    ref = _reference_root()
    if ref is None:
        pytest.skip("the reference package is not on this machine")
    ours = _our_names(ROOT / "trainscale_b200")
    missing = {n: f for n, f in _public_defs(ref).items() if n not in ours}
    assert not missing, f"{len(missing)} names without a counterpart: {sorted(missing.items())[:20]}"


def test_every_module_of_the_package_imports():
    """The surface tests skip modules that fail to import, so a broken import must fail on its own."""
    import importlib
    import pkgutil

    import trainscale_b200
    failed = {}
    for m in pkgutil.walk_packages(trainscale_b200.__path__, "trainscale_b200."):
        if m.name.endswith("__main__"):
            continue
        try:
            importlib.import_module(m.name)
        except Exception as e:   # noqa: BLE001
            failed[m.name] = repr(e)[:120]
    assert not failed, failed


def _reference_methods(root: Path) -> dict[str, set[str]]:
    """{class name: public method names} over every module-level class of the reference (same-named classes of
    different files are merged)."""
    out: dict[str, set[str]] = {}
    for p in root.rglob("*.py"):
        if "examples" in p.parts:
            continue
        try:
            tree = ast.parse(p.read_text())
        except SyntaxError:
            continue
        for node in tree.body:
            if isinstance(node, ast.ClassDef):
                out.setdefault(node.name, set()).update(
                    n.name for n in node.body
                    if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)) and not n.name.startswith("_"))
    return out


def _our_classes() -> dict[str, set]:
    import importlib
    import inspect
    import pkgutil

    import trainscale_b200
    found: dict[str, set] = {}
    for m in pkgutil.walk_packages(trainscale_b200.__path__, "trainscale_b200."):
        if m.name.endswith("__main__"):
            continue
        try:
            mod = importlib.import_module(m.name)
        except Exception:   # noqa: BLE001 - optional dependencies of single modules
            continue
        for n, v in vars(mod).items():
            if inspect.isclass(v) and v.__module__.startswith("trainscale_b200"):
                found.setdefault(n, set()).add(v)
    return found


def _has_member(cls, name: str) -> bool:
    import inspect
    if hasattr(cls, name) or name in getattr(cls, "__annotations__", {}) or name in getattr(cls, "__dataclass_fields__", {}):
        return True
    try:                                              # attributes that exist per instance (set in __init__)
        src = inspect.getsource(cls)
    except (OSError, TypeError):
        return False
    return any(f"self.{name}{tail}" in src for tail in (" =", "=", ",", " :")) or f", self.{name}" in src


def test_every_public_method_of_a_shared_class_exists_here():
    """For every class that exists under the same name on both sides, each public method / property of the reference's
    class is an attribute of ours (a method, a property, a field or an alias)."""
    ref = _reference_root()
    if ref is None:
        pytest.skip("the reference package is not on this machine")
    ours = _our_classes()
    missing = {}
    for cname, methods in _reference_methods(ref).items():
        if cname not in ours:
            continue
        lack = sorted(m for m in methods if not any(_has_member(c, m) for c in ours[cname]))
        if lack:
            missing[cname] = lack
    assert not missing, f"{sum(map(len, missing.values()))} members missing: {sorted(missing.items())[:15]}"


def _reference_function_params(root: Path) -> dict[str, list[list[str]]]:
    out: dict[str, list[list[str]]] = {}
    for p in root.rglob("*.py"):
        if "examples" in p.parts:
            continue
        try:
            tree = ast.parse(p.read_text())
        except SyntaxError:
            continue
        for node in tree.body:
            if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)) and not node.name.startswith("_"):
                a = node.args
                out.setdefault(node.name, []).append([x.arg for x in a.posonlyargs + a.args + a.kwonlyargs])
    return out


def test_shared_functions_take_the_reference_keyword_names():
    """For every public function that exists under the same name on both sides, ours can be called with each of the
    reference's parameter names as a keyword (its own parameter, an alias, or **kwargs)."""
    import importlib
    import inspect
    import pkgutil

    import trainscale_b200
    ref = _reference_root()
    if ref is None:
        pytest.skip("the reference package is not on this machine")
    ours: dict[str, set] = {}
    for m in pkgutil.walk_packages(trainscale_b200.__path__, "trainscale_b200."):
        if m.name.endswith("__main__"):
            continue
        try:
            mod = importlib.import_module(m.name)
        except Exception:   # noqa: BLE001
            continue
        for n, v in vars(mod).items():
            if not n.startswith("_") and callable(v) and not inspect.isclass(v) \
                    and getattr(v, "__module__", "").startswith("trainscale_b200"):
                ours.setdefault(n, set()).add(v)

    def lacking(fn, names):
        try:
            ps = inspect.signature(fn).parameters
        except (ValueError, TypeError):
            return []
        if any(p.kind is p.VAR_KEYWORD for p in ps.values()):
            return []
        return [n for n in names if n not in ps]

    missing = {}
    for name, variants in _reference_function_params(ref).items():
        if name not in ours:
            continue
        best = min((lacking(fn, names) for names in variants for fn in ours[name]), key=len)
        if best:
            missing[name] = best
    assert not missing, f"{len(missing)} functions lack reference keywords: {sorted(missing.items())[:15]}"


def test_last_helpers_behave():
    import torch

    from trainscale_b200 import benchmark_suite as BS
    from trainscale_b200.core.types import Err, Ok
    from trainscale_b200.data import length_manager as LM
    from trainscale_b200.data import packing as P
    from trainscale_b200.data import prompt_engine as PE
    from trainscale_b200.data import tokenization as TK
    from trainscale_b200.parallel import activation as A
    from trainscale_b200.parallel import cp as C
    from trainscale_b200.parallel import dist_utils as U
    from trainscale_b200.trainer import base as B
    from trainscale_b200.trainer.sota_trainer import SOTATrainer, create_trainer_from_config
    m = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU(), torch.nn.Linear(4, 4))
    ref = m(torch.ones(2, 4)).detach()
    A.wrap_activation_checkpointing(m, torch.nn.Linear)
    x = torch.ones(2, 4, requires_grad=True)
    y = m(x)
    y.sum().backward()
    assert torch.allclose(y, ref) and x.grad is not None and m[0]._ts_checkpointed
    g = A.OffloadTensorGroup("mlp")
    g.add("h", torch.arange(6.0).view(2, 3))
    assert g.offload_all(A.OffloadTarget.CPU_PAGED) == 24 and torch.equal(g.get("h"), torch.arange(6.0).view(2, 3))
    assert A.ActivationOffloadConfig(min_offload_tensor_size=1024).build().min_bytes == 2048
    with U.no_sync(m):
        pass
    U.allreduce_conditional_embedding_grads(m, None)                  # no pipeline group: nothing to do
    assert LM.saturating_sub(3, 5) == 0 and LM.clamp(7, 0, 5) == 5 and LM.is_tokenizer(TK.ByteTokenizer())
    assert P.calculate_packing_efficiency([3, 4, 5], [[0, 1], [2]], 8) == 0.75
    assert TK.ensure_tokenizer_padding(TK.ByteTokenizer()) >= 0
    oks, errs = PE.extract_successful([Ok(1), Err(ValueError("x")), Ok(2)])
    assert oks == [1, 2] and isinstance(errs[0], ValueError)
    out = B.TrainOutput.from_summary({"global_step": 3, "train_loss": 1.25})
    assert out.global_step == 3 and "1.250000" in repr(out) and B.PredictionOutput(torch.zeros(1)).label_ids is None
    s = C.BalancerStrategy("head_tail")
    t = torch.arange(16).view(1, 16)
    parts = [s.partition(t, r, 2, 1) for r in range(2)]
    assert parts[0].tolist() == [[0, 1, 2, 3, 12, 13, 14, 15]] and torch.equal(s.unpartition(parts, 1), t)
    row = BS.BenchmarkResult.from_row({"name": "k", "ms": 1.0, "baseline_ms": 2.0, "gbs": 100.0})
    assert row.speedup == 2.0 and row.baseline_metric == 50.0 and row.metric_name == "GB/s"
    tr = create_trainer_from_config({"model": {"architecture": "llama-tiny"},
                                     "hardware": {"device": "cpu", "precision": "fp32"},
                                     "distributed": {"enabled": False}})
    assert isinstance(tr, SOTATrainer)


def _reference_method_params(root: Path) -> dict[tuple[str, str], list[list[str]]]:
    """{(class, method): [parameter names of each definition]} for constructors and public methods of the reference's
    module-level classes.  `forward` / `backward` of autograd functions are left out: `Function.apply` passes their
    arguments by position, so their parameter names are not part of any call."""
    out: dict[tuple[str, str], list[list[str]]] = {}
    for p in root.rglob("*.py"):
        if "examples" in p.parts:
            continue
        try:
            tree = ast.parse(p.read_text())
        except SyntaxError:
            continue
        for node in tree.body:
            if not isinstance(node, ast.ClassDef) or node.name.startswith("_"):
                continue
            bases = {getattr(b, "attr", getattr(b, "id", "")) for b in node.bases}
            for n in node.body:
                if not isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)):
                    continue
                if n.name.startswith("_") and n.name != "__init__":
                    continue
                decorators = {getattr(d, "id", getattr(d, "attr", "")) for d in n.decorator_list}
                if "property" in decorators or "setter" in decorators:
                    continue
                if "Function" in bases and n.name in ("forward", "backward"):
                    continue
                a = n.args
                names = [x.arg for x in a.posonlyargs + a.args + a.kwonlyargs if x.arg not in ("self", "cls")]
                out.setdefault((node.name, n.name), []).append(names)
    return out


def test_shared_methods_take_the_reference_keyword_names():
    """For every class that exists under the same name on both sides, the constructor and each public method of ours
    can be called with every parameter name of the reference's as a keyword."""
    import inspect

    ref = _reference_root()
    if ref is None:
        pytest.skip("the reference package is not on this machine")
    ours = _our_classes()

    def lacking(fn, names):
        if fn is None or isinstance(fn, property):
            return []
        try:
            ps = inspect.signature(fn).parameters
        except (ValueError, TypeError):
            return []
        if any(p.kind is p.VAR_KEYWORD for p in ps.values()):
            return []
        return [n for n in names if n not in ps]

    missing = {}
    for (cname, mname), variants in _reference_method_params(ref).items():
        if cname not in ours:
            continue
        targets = [c if mname == "__init__" else inspect.getattr_static(c, mname, None) for c in ours[cname]]
        targets = [getattr(t, "__func__", t) for t in targets if t is not None]
        if not targets:
            continue
        best = min((lacking(fn, names) for names in variants for fn in targets), key=len)
        if best:
            missing[f"{cname}.{mname}"] = best
    assert not missing, f"{len(missing)} methods lack reference keywords: {sorted(missing.items())[:15]}"


def _our_modules():
    import importlib
    import pkgutil

    import trainscale_b200
    mods = []
    for m in pkgutil.walk_packages(trainscale_b200.__path__, "trainscale_b200."):
        if m.name.endswith("__main__"):
            continue
        try:
            mods.append(importlib.import_module(m.name))
        except Exception:   # noqa: BLE001
            continue
    return mods


def test_module_level_constants_and_aliases_of_the_reference_exist_here():
    """Annotated constants (`X: Final[int] = 64`), plain module-level assignments and `import ... as alias` re-exports
    of the reference's modules have a counterpart of the same name in some module of this package (type variables with
    one-letter names and loggers aside)."""
    ref = _reference_root()
    if ref is None:
        pytest.skip("the reference package is not on this machine")
    wanted: dict[str, str] = {}
    for p in ref.rglob("*.py"):
        if "examples" in p.parts:
            continue
        try:
            tree = ast.parse(p.read_text())
        except SyntaxError:
            continue
        for node in tree.body:
            names: list[str] = []
            if isinstance(node, ast.AnnAssign) and isinstance(node.target, ast.Name) and node.value is not None:
                names = [node.target.id]
            elif isinstance(node, ast.Assign):
                names = [t.id for t in node.targets if isinstance(t, ast.Name)]
            elif isinstance(node, ast.ImportFrom):
                names = [a.asname for a in node.names if a.asname and a.asname != a.name]
            for n in names:
                if not n.startswith("_") and len(n) > 1 and n != "logger":
                    wanted.setdefault(n, str(p.relative_to(ref)))
    mods = _our_modules()
    missing = {n: f for n, f in wanted.items() if not any(hasattr(m, n) for m in mods)}
    assert not missing, f"{len(missing)} module-level names without a counterpart: {sorted(missing.items())[:20]}"


def test_the_reference_import_paths_resolve():
    """With `trainscale_b200.reference_paths` imported, every absolute `from data_pipeline... import name` statement
    found anywhere in the reference (its examples included) resolves to an object of this package - for every name the
    reference itself still defines (two of its older example scripts import names that no longer exist there)."""
    import importlib

    ref = _reference_root()
    if ref is None:
        pytest.skip("the reference package is not on this machine")
    import trainscale_b200.reference_paths as paths
    if not paths.install():
        pytest.skip("a real data_pipeline package is importable here")
    defined: set[str] = set()
    pairs: dict[tuple[str, str], str] = {}
    for p in ref.rglob("*.py"):
        try:
            tree = ast.parse(p.read_text())
        except SyntaxError:
            continue
        for node in ast.walk(tree):
            if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
                defined.add(node.name)
            elif isinstance(node, ast.Assign):
                defined.update(t.id for t in node.targets if isinstance(t, ast.Name))
            elif isinstance(node, ast.AnnAssign) and isinstance(node.target, ast.Name):
                defined.add(node.target.id)
            elif isinstance(node, ast.ImportFrom):
                defined.update(a.asname for a in node.names if a.asname)
                if node.level == 0 and node.module and node.module.split(".")[0] == "data_pipeline":
                    for a in node.names:
                        if a.name != "*" and not a.name.startswith("_"):
                            pairs.setdefault((node.module, a.name), str(p.relative_to(ref)))
    modules = {m for m, _ in pairs}
    failed = {}
    for (module, name), where in pairs.items():
        is_submodule = f"{module}.{name}" in modules or any(m.startswith(f"{module}.{name}.") for m in modules)
        if name not in defined and not is_submodule:
            continue
        try:
            getattr(importlib.import_module(module), name)
        except Exception as e:   # noqa: BLE001
            failed[f"{module}:{name}"] = f"{where}: {e!r}"[:160]
    assert len(pairs) > 500 and not failed, f"{len(failed)} of {len(pairs)} imports fail: {sorted(failed.items())[:10]}"
    # spot checks: the path selects the right one of several same-named objects
    from data_pipeline.trainer.distributed.context_parallel import CUDATimer as cp_timer
    from data_pipeline.trainer.distributed.ddp import CUDATimer as ddp_timer
    from data_pipeline.trainer.kernels import flash_attention
    import trainscale_b200.kernels as K
    import trainscale_b200.parallel.ddp as ddp
    assert ddp_timer is ddp.CUDATimer and cp_timer is not None
    # a function whose positional conventions differ resolves to its variant with the reference's conventions
    assert flash_attention is K.flash_attention.__reference_form__
    from data_pipeline.trainer import inference
    import trainscale_b200.inference as ours_inference
    assert inference is ours_inference


def test_a_script_in_the_reference_style_runs_through_the_reference_paths():
    """The calls a user script of the reference typically makes (optimizer steps, schedulers, losses, metric
    collection, a tensor-parallel layer on one rank, attention in the reference's layout, gradient clipping, the compiler
    facade), written against `data_pipeline...` imports and run on this package."""
    import torch
    import torch.nn as nn

    import trainscale_b200.reference_paths as paths
    if not paths.install():
        pytest.skip("a real data_pipeline package is importable here")
    from data_pipeline.trainer import (AdaFactor, AdamW, CosineScheduler, CrossEntropyLoss, DeviceManager, FocalLoss, LAMB,
                                       TrainingArguments, clip_grad_norm_, is_main_process)
    from data_pipeline.trainer.distributed import ColumnParallelLinear
    from data_pipeline.trainer.distributed.expert_parallel import ExpertParallelConfig, MoELayer
    from data_pipeline.trainer.kernels import compile_model, flash_attention
    from data_pipeline.trainer.metrics import Accuracy, F1Score, MetricCollection

    torch.manual_seed(0)
    for make in (lambda p: AdamW(p, lr=1e-3), lambda p: LAMB(p, lr=1e-3), lambda p: AdaFactor(p, lr=1e-3)):
        model = nn.Linear(64, 10)
        before = model.weight.detach().clone()
        opt = make(model.parameters())
        model(torch.randn(4, 64)).sum().backward()
        opt.step()
        assert not torch.equal(before, model.weight.detach())
    opt = torch.optim.Adam(nn.Linear(4, 4).parameters(), lr=1e-3)
    sched = CosineScheduler(opt, num_training_steps=100, warmup_steps=10)
    lrs = []
    for _ in range(100):
        sched.step()
        lrs.append(sched.get_last_lr()[0])
    assert max(lrs) == pytest.approx(1e-3, rel=1e-3) and lrs[-1] < lrs[50] < lrs[11]
    logits, targets = torch.randn(32, 10), torch.randint(0, 10, (32,))
    assert CrossEntropyLoss(label_smoothing=0.1)(logits, targets).item() > 0 and FocalLoss(gamma=2.0)(logits, targets).item() > 0
    collection = MetricCollection([Accuracy(), F1Score(average="macro")])
    collection.update(torch.randn(100, 5), torch.randint(0, 5, (100,)))
    results = collection.compute()
    assert 0.0 <= results["accuracy"] <= 1.0 and "f1" in results
    assert ColumnParallelLinear(64, 128)(torch.randn(4, 64)).shape == (4, 128)
    out, aux, _ = MoELayer(ExpertParallelConfig(num_experts=4, top_k=2, hidden_size=64, intermediate_size=128))(
        hidden_states=torch.randn(2, 8, 64))
    assert out.shape == (2, 8, 64) and aux.dim() == 0
    q = torch.randn(2, 4, 16, 32)
    k, v = torch.randn_like(q), torch.randn_like(q)
    want = nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert torch.allclose(flash_attention(q, k, v, causal=True), want, atol=1e-5)     # [batch, heads, seq, dim], as there
    assert DeviceManager.auto_detect().device is not None and is_main_process()
    model = nn.Linear(64, 10)
    model(torch.randn(4, 64)).sum().backward()
    clip_grad_norm_(model.parameters(), max_norm=1.0)
    assert float(torch.nn.utils.clip_grad_norm_(model.parameters(), float("inf"))) <= 1.0 + 1e-4
    assert compile_model(model, mode="default")(torch.randn(4, 64)).shape == (4, 10)
    assert TrainingArguments(output_dir="out").output_dir == "out"


def test_soft_capped_attention_by_position_through_the_reference_paths():
    """`slow_attention_softcapping(Q, K, V, causal_mask, config, bsz, q_len)` and its two siblings, called by position
    with [batch, heads, seq, dim] tensors as the reference's callers do, against the formula written out."""
    import torch

    import trainscale_b200.reference_paths as paths
    if not paths.install():
        pytest.skip("a real data_pipeline package is importable here")
    from data_pipeline.trainer.kernels.flex_attention import (FlexAttentionConfig, attention_softcapping_compiled,
                                                              inference_attention_single_token,
                                                              slow_attention_softcapping)
    torch.manual_seed(0)
    cfg = FlexAttentionConfig(num_attention_heads=4, num_key_value_heads=2, head_dim=8, query_pre_attn_scalar=8,
                              attn_logit_softcapping=30.0)
    Q, K, V = torch.randn(1, 4, 6, 8), torch.randn(1, 2, 6, 8), torch.randn(1, 2, 6, 8)
    mask = torch.zeros(6, 6).masked_fill(torch.ones(6, 6, dtype=torch.bool).triu(1), float("-inf"))
    scores = (Q @ K.repeat_interleave(2, 1).transpose(-1, -2)) * 8 ** -0.5
    want = (torch.softmax(30 * torch.tanh(scores / 30) + mask, -1) @ V.repeat_interleave(2, 1)).transpose(1, 2).reshape(1, 6, 32)
    assert torch.allclose(slow_attention_softcapping(Q, K, V, mask, cfg, 1, 6), want, atol=1e-5)
    assert torch.allclose(attention_softcapping_compiled(Q, K, V, mask, 8.0, 30.0, 4, 2, 8), want, atol=1e-5)
    last = inference_attention_single_token(Q[:, :, -1:], K, V, cfg)                 # the last query sees every key
    assert torch.allclose(last, want[:, -1:], atol=1e-5)
