"""Behaviour of the members that classes share with the reference by name: builders, tokenizer wrapper, DDP engine
records, training configuration, serving engines, hub manager, length manager, callbacks, LoRA layer, trainer."""
import asyncio
import os

import pytest
import torch
import torch.nn as nn


def test_dataloader_builder_fluent_chain():
    from trainscale_b200.data.dataloader_factory import DataLoaderBuilder
    ds = [{"input_ids": torch.arange(n + 1), "labels": torch.arange(n + 1)} for n in range(10)]
    dl = (DataLoaderBuilder().with_dataset(ds).with_batch_size(4).with_shuffle(False).with_seed(3).with_num_workers(0)
          .with_pin_memory(False).with_drop_last(True).with_padding(pad_token_id=7, label_pad_token_id=-100).build())
    batches = list(dl)
    assert len(batches) == 2                                  # 10 rows, batch 4, last dropped
    b = batches[0]
    assert b["input_ids"].shape == (4, 4) and b["input_ids"][0, 1:].tolist() == [7, 7, 7]
    assert b["labels"][0, 1:].tolist() == [-100, -100, -100]


def test_tokenizer_wrapper_vocabulary_members():
    from trainscale_b200.data.tokenization import ByteTokenizer, TokenizerWrapper
    w = TokenizerWrapper(ByteTokenizer())
    assert len(w) == w.vocab_size and w.original_vocab_size <= w.vocab_size
    assert w.num_added_tokens == w.vocab_size - w.original_vocab_size
    assert w.vocab_was_modified == (w.num_added_tokens > 0)
    ids = w.encode_raw("hi there")
    assert w.decode_batch([ids, ids]) == [w.decode(ids)] * 2
    toks = w.convert_ids_to_tokens(list(ids))
    assert w.convert_tokens_to_ids(toks) == list(ids)
    info = w.get_special_tokens_info()
    assert set(w.get_all_special_token_ids()) >= {v for v in (info.get("pad_token_id"), info.get("eos_token_id"))
                                                   if v is not None}


def test_ddp_metrics_and_pressure_monitor():
    from trainscale_b200.parallel.ddp import DDPMetrics, MemoryPressureMonitor
    m = DDPMetrics()
    for _ in range(4):
        m.record_allreduce(4 * 10 ** 9, 2.0)
        m.steps += 1
    assert m.compute_avg_latency_ms() == pytest.approx(2.0)
    assert m.compute_bandwidth_gbps() == pytest.approx(16 / 0.008)
    m.reset()
    assert m.steps == 0 and m.compute_avg_latency_ms() == 0.0 and m.compute_bandwidth_gbps() == 0.0
    used = [10]
    mon = MemoryPressureMonitor(probe=lambda: (used[0], 100))
    assert mon.get_pressure_level() == 0
    used[0] = 90
    assert mon.get_pressure_level() == 1
    used[0] = 99
    assert mon.get_pressure_level() == 2
    assert mon.allocated_bytes >= 0 and mon.reserved_bytes >= 0 and mon.emergency_free() >= 0


def test_training_config_reference_fields_and_aliases():
    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.config.training_args import TrainingConfig, TrainingMode, get_qlora_config
    c = TrainingConfig(model_name="tiny", batch_size=2, gradient_accumulation_steps=4)
    assert c.model_name_or_path == "tiny" and c.per_device_train_batch_size == 2
    assert c.effective_batch_size == 8
    q = get_qlora_config("tiny", r=8)
    assert q.training_mode == TrainingMode.QLORA and q.load_in_4bit and q.to_lora_config().r == 8
    assert q.to_quant_config().load_in_4bit
    again = TrainingConfig.from_dict(q.to_dict())
    assert again.to_dict() == q.to_dict()
    s = SOTAConfig.from_dict(q.to_sota_dict())
    assert s.lora.enabled and s.lora.r == 8


def _cpu_engine_config(preset):
    preset.device = "cpu"
    preset.cache.num_gpu_blocks = 64
    return preset


def test_engine_presets_profiles():
    from trainscale_b200.inference.engine import EnginePresets
    hi, lo = EnginePresets.high_throughput_batch("tiny"), EnginePresets.low_latency_interactive("tiny")
    assert hi.scheduler.max_num_seqs > lo.scheduler.max_num_seqs
    assert hi.scheduler.max_num_batched_tokens > lo.scheduler.max_num_batched_tokens
    sp = EnginePresets.speculative_fast_decode("tiny", draft_model="tiny", num_speculative_tokens=3)
    assert sp.speculative.enabled and sp.speculative.num_speculative_tokens == 3
    assert EnginePresets.quantized_memory_efficient("tiny", "fp8").quantization.method == "fp8"
    big = EnginePresets.multi_gpu_large_model("tiny", tp_size=4, pp_size=2)
    assert big.parallel.tensor_parallel_size == 4 and big.parallel.pipeline_parallel_size == 2
    ml = EnginePresets.multi_lora_serving("tiny", max_lora_rank=32, max_concurrent_loras=2)
    assert ml.lora.enabled and ml.lora.max_loras == 2 and ml.lora.max_lora_rank == 32


def test_generate_with_lora_loads_adapter_directory(tmp_path):
    from trainscale_b200 import lora as L
    from trainscale_b200.inference.engine import EnginePresets, GenerationParams, SOTAInferenceEngine
    from trainscale_b200.models.llama import build_model
    m = L.get_peft_model(build_model("tiny", dtype=torch.float32, device="cpu", seed=0), L.LoraConfig(r=4))
    e = SOTAInferenceEngine(_cpu_engine_config(EnginePresets.multi_lora_serving("tiny")), model=m)
    gp = GenerationParams(max_tokens=4, temperature=0.0)
    base = e.generate_single("hello", gp).unwrap().token_ids
    for n, p in m.named_parameters():
        if "lora_B" in n:
            nn.init.normal_(p, std=0.5)
    L.save_adapter(m, tmp_path)
    for n, p in m.named_parameters():                     # the model itself goes back to a no-op adapter
        if "lora_B" in n:
            nn.init.zeros_(p)
    tuned = e.generate_with_lora("hello", "a1", str(tmp_path), params=gp).unwrap().token_ids
    assert tuned != base
    assert e.generate_single("hello", gp).unwrap().token_ids == base        # requests without an adapter are unchanged
    assert e.generate_with_lora("hello", "a1", params=gp).unwrap().token_ids == tuned   # found by name the second time
    assert e.generate_with_lora("x", "unknown").is_err()
    assert e.get_metrics_summary()["requests"] == 4 and e.engine is e.core and e.metrics is e.core.metrics


def test_async_engine_generate_batch_and_shutdown():
    from trainscale_b200.inference.engine import (EnginePresets, GenerationParams, SOTAAsyncStreamEngine,
                                                  SOTAInferenceEngine)
    cfg = _cpu_engine_config(EnginePresets.low_latency_interactive("tiny"))
    gp = GenerationParams(max_tokens=3, temperature=0.0)
    a = SOTAAsyncStreamEngine(cfg)
    sync_ids = SOTAInferenceEngine(cfg, model=a.core.model).generate_single("abc", gp).unwrap().token_ids

    async def main():
        one = (await a.generate("abc", gp)).unwrap()
        many = (await a.generate_batch(["a", "bb", "ccc"], gp)).unwrap()
        assert a.active_request_count == 0
        await a.shutdown()
        return one, many

    one, many = asyncio.run(main())
    assert one.token_ids == sync_ids and len(many) == 3 and all(len(r.token_ids) == 3 for r in many)
    assert a.get_metrics_summary()["requests"] == 4


def test_request_metrics_marks():
    from trainscale_b200.inference.engine import RequestMetrics
    m = RequestMetrics("r")
    m.mark_submitted()
    m.mark_first_token()
    first = m.first_token
    m.mark_first_token()
    assert m.first_token == first                         # only the first call counts
    m.mark_complete(5)
    assert m.completion_tokens == 5 and m.e2e >= m.ttft >= 0 and m.tpot is not None


def test_hub_manager_round_trip_through_a_local_folder(tmp_path):
    from trainscale_b200.hub import HubConfig, HubErrorCode, HubManager, ModelSerializer
    src, dst = nn.Linear(64, 64), nn.Linear(64, 64)
    h = HubManager(HubConfig(repo_id="someone/model", token="", shard_size_bytes=8 * 1024))
    seen = []
    r = h.push_to_hub(src, local_dir=tmp_path, progress_callback=lambda a, b: seen.append((a, b)))
    # no network / token here: the upload itself fails with a classified error, the folder is complete
    assert r.is_err() and r.error.context["code"] == HubErrorCode.DEPENDENCY_MISSING
    assert (tmp_path / "README.md").exists() and seen and seen[0][0] == 0
    assert h.load_from_hub(dst, str(tmp_path)).is_ok()
    assert torch.equal(src.weight, dst.weight) and torch.equal(src.bias, dst.bias)
    assert h.get_metrics()["uploads_failed"] >= 1 and h.config.repo_id == "someone/model"
    assert HubManager().push_to_hub(src).error.context["code"] == HubErrorCode.VALIDATION_ERROR
    assert HubManager().pull_from_hub().is_err()
    ser = ModelSerializer(8 * 1024)
    res = ser.serialize(src, tmp_path / "again").unwrap()
    assert res.total_bytes > 0 and len(res.shards) >= 1 and isinstance(ser.safetensors_available, bool)


def test_length_manager_column_limits():
    from trainscale_b200.data.length_manager import (ColumnLengthConfig, LengthManager, LengthManagerConfig,
                                                     TokenEstimator)
    lm = LengthManager(LengthManagerConfig(max_total_length=64, per_column={"a": ColumnLengthConfig("a", max_length=5)}))
    assert lm.max_length == 64 and lm.padding_strategy == lm.config.padding_strategy
    assert lm.get_column_config("a").max_tokens == 5 and lm.get_column_config("zzz").max_tokens is None
    lm.set_column_config("b", ColumnLengthConfig(max_chars=7))
    assert lm.preprocess_text("hello world this is long", "b") == "hello w"
    assert len(lm.preprocess_text("x" * 100, "a")) == lm.estimator.tokens_to_chars(5)
    assert lm.preprocess_text("x" * 100, "a", max_chars=3) == "xxx"          # the explicit limit wins
    assert len(lm.preprocess_text("y" * 1000)) == lm.estimator.tokens_to_chars(64)
    assert lm.preprocess_text("", "a") == ""
    te = TokenEstimator(chars_per_token=4.0)
    assert te.estimate_tokens("") == 0 and te.estimate_tokens("abcdefgh") == 2 and te.tokens_to_chars(10) == 40

    class Tok:
        def encode(self, text):
            return text.split()
    assert TokenEstimator(Tok()).estimate_tokens("a b c") == 3


def test_callback_handler_trigger_stops_at_should_stop():
    from trainscale_b200.callbacks import Callback, CallbackContext, CallbackHandler
    calls = []

    class A(Callback):
        order = 0
        def on_step_end(self, ctx):
            calls.append("a")
            ctx.should_stop = True

    class B(Callback):
        order = 1
        def on_step_end(self, ctx):
            calls.append("b")

    h = CallbackHandler()
    h.add_callback(B())
    h.add_callback(A())
    h.set_trainer("trainer")
    assert all(c.trainer == "trainer" for c in h.callbacks) and h.callbacks[0].priority == 0
    h.trigger("on_step_end", CallbackContext())
    assert calls == ["a"]                                  # B is skipped once A asked to stop
    h.fire("on_step_end", CallbackContext())
    assert calls == ["a", "a", "b"]
    h.remove_callback(A)
    assert [type(c) for c in h.callbacks] == [B]
    with pytest.raises(ValueError):
        h.trigger("no_such_hook", CallbackContext())


def test_lora_linear_from_linear_and_merge():
    from trainscale_b200.lora import LoRALinear
    torch.manual_seed(0)
    lin = nn.Linear(16, 8)
    m = LoRALinear.from_linear(lin, r=4, lora_alpha=8)
    x = torch.randn(3, 16)
    assert torch.allclose(m(x), lin(x), atol=1e-6)          # B = 0: identical to the base layer
    nn.init.normal_(m.lora_B)
    assert not torch.allclose(m(x), lin(x), atol=1e-3)
    assert torch.allclose(m(x), x @ m.merge_weights().T + lin.bias, atol=1e-5)
    assert not m.weight.requires_grad and m.lora_A.requires_grad
    m.reset_lora_parameters()
    assert float(m.lora_B.detach().abs().sum()) == 0.0
    with pytest.raises(ValueError):
        LoRALinear(16, 8).merge_weights()


def test_trainer_builds_loaders_from_datasets_and_reloads_weights(tmp_path):
    from trainscale_b200.config.training_args import TrainingArguments
    from trainscale_b200.core.errors import ConfigurationError
    from trainscale_b200.trainer.base import Trainer

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(4, 1)

    args = TrainingArguments(per_device_train_batch_size=4, gradient_accumulation_steps=2, world_size=8,
                             num_train_epochs=1, output_dir=str(tmp_path))
    assert args.effective_batch_size == 64 and args.output_path == tmp_path
    with pytest.raises(ValueError):
        TrainingArguments(push_to_hub=True)
    ds = [{"x": torch.randn(4), "y": torch.randn(1)} for _ in range(16)]
    t = Trainer(M(), args, train_dataset=ds, eval_dataset=ds,
                compute_loss=lambda m, b: ((m.l(b["x"]) - b["y"]) ** 2).mean())
    assert len(t.get_train_dataloader()) == 4 and len(t.get_eval_dataloader()) == 2
    first = [b["x"] for b in t.get_train_dataloader()]
    assert all(torch.equal(a, b) for a, b in zip(first, [b["x"] for b in t.get_train_dataloader()]))   # seeded shuffle
    assert t.train()["global_step"] == 2
    t.save_model(str(tmp_path / "w"))
    w = t.model.l.weight.detach().clone()
    nn.init.zeros_(t.model.l.weight)
    t.load_model(str(tmp_path / "w"))
    assert torch.equal(w, t.model.l.weight)
    with pytest.raises(ConfigurationError):
        Trainer(M(), args).get_train_dataloader()


def test_preprocessed_dataset_select_and_stage_splits():
    from trainscale_b200.config.data_schema import SplitSpec, StageConfig
    from trainscale_b200.data.dataset_wrappers import PreprocessedDataset

    class Ex:
        def __init__(self, row):
            self.row = row
        def to_dict(self):
            return {"input_ids": [self.row["v"]]}

    class Engine:
        calls = 0
        def process(self, row):
            Engine.calls += 1
            return Ex(row)

    d = PreprocessedDataset([{"v": i} for i in range(6)], Engine())
    assert int(d[2]["input_ids"][0]) == 2 and int(d[2]["input_ids"][0]) == 2 and Engine.calls == 1   # second read cached
    d.clear_cache()
    d[2]
    assert Engine.calls == 2 and d.features is None
    sub = d.select([4, 1])
    assert len(sub) == 2 and int(sub[0]["input_ids"][0]) == 4
    st = StageConfig("s1", {"extra": SplitSpec("extra"), "train": SplitSpec("train")})
    assert list(st.all_splits()) == ["train", "extra"] and st.get_split("train") is st.train and st.get_split("nope") is None


def test_registry_incremental_registration_and_reports():
    from trainscale_b200.models.llama import build_model
    from trainscale_b200.registry import (MODEL_REGISTRY, Capability, DependencyGraph, HardwareCapability, KernelPatcher,
                                          ModelInfo, ModuleContract, RegistryValidator)
    from trainscale_b200.registry.catalog import BaseModuleContract
    cpu = HardwareCapability("cpu", (0, 0), 0, 0.0, frozenset())
    b200 = HardwareCapability("b200", (10, 0), 148, 180.0, frozenset(Capability))
    v = RegistryValidator(hardware=b200)
    assert v.register(ModuleContract("gemm_torch")).is_ok()
    assert v.register(ModuleContract("gemm_tcgen05", (Capability.TCGEN05,), fallback="gemm_torch")).is_ok()
    assert v.register(ModuleContract("attn", (Capability.TCGEN05,), ("gemm_tcgen05",))).is_ok()
    missing = v.register(ModuleContract("x", (), ("nope",)))
    assert missing.is_err() and missing.error.missing_deps == ("nope",)
    assert v.register(ModuleContract("attn")).error.reason == "duplicate_registration"
    order = v.get_registration_order().unwrap()
    assert order.index("gemm_tcgen05") < order.index("attn")
    rep = v.get_capabilities_report()
    assert rep["total_registered"] == 3 and rep["validation_failed"] == 0 and "tcgen05" in rep["hardware_capabilities"]
    off_gpu = RegistryValidator(v.matrix, cpu)
    rep = off_gpu.get_capabilities_report()
    assert rep["available_kernels"] == ["gemm_torch"] and rep["validation_failed"] == 2
    assert off_gpu.validate_contract(ModuleContract("needs_fp8", (Capability.FP8,))).is_err()
    assert v.matrix.get_optimal_kernel("gemm_tcgen05", cpu).name == "gemm_torch"
    assert v.matrix.get_optimal_kernel("gemm_tcgen05", b200).name == "gemm_tcgen05"
    b = BaseModuleContract("b", (2, 1, 0), frozenset(), frozenset({Capability.FP8}))
    assert b.version_string() == "2.1.0" and b.get_fallback() is None
    assert v.matrix.register_kernel(b, ["gemm_torch"]).is_ok()
    assert v.matrix.get_optimal_kernel("b", cpu).name == "gemm_torch" and "b" in v.matrix.get_all_kernels()
    assert "b" in v.matrix.get_available_kernels(b200) and "b" not in v.matrix.get_available_kernels(cpu)

    g = DependencyGraph()
    g.add_module("a", {"b"})
    assert g.validate_dependencies("a").error.missing_deps == ("b",)
    g.add_module("b", {"a"})
    assert g.topological_sort().is_err() and g.get_dependencies("a") == frozenset({"b"})
    g.remove_module("b")
    assert g.topological_sort().unwrap() == ["b", "a"] and g.validate_dependencies("a").is_err()

    mc = ModuleContract("k", (Capability.FP8,), ("d",), "f")
    assert mc.validate(cpu).is_err() and mc.validate(b200).is_ok() and mc.get_fallback() == "f"
    assert mc.dependencies == frozenset({"d"}) and mc.hardware_requirements == frozenset({Capability.FP8})
    assert ModelInfo.construct_model_name("Llama", "3.1", "8", instruct_tag="Instruct") == "Llama-3.1-8B-Instruct"
    assert MODEL_REGISTRY["llama"].model_path == "meta-llama/llama"
    stats = KernelPatcher().get_stats(build_model("tiny", dtype=torch.float32, device="cpu"))
    assert stats["attention_total"] == stats["attention_patched"] > 0 and stats["mlp_total"] == stats["mlp_patched"] > 0

    class Foreign(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = nn.LayerNorm(8)

    assert KernelPatcher().get_stats(Foreign()) == {**{k: 0 for k in stats}, "layernorm_total": 1}


def test_attention_config_and_backend_capabilities():
    from trainscale_b200.kernels import (AttentionBackend, AttentionMaskType, BackendCapabilities, FlashAttentionConfig,
                                         FlexAttentionConfig)
    c = FlashAttentionConfig(head_dim=64, num_heads=8, num_kv_heads=2)
    assert c.scale == 0.125 and c.num_kv_groups == 4 and c.is_gqa and c.mask_type is AttentionMaskType.CAUSAL
    assert FlashAttentionConfig(softmax_scale=0.5).scale == 0.5
    assert FlashAttentionConfig(sliding_window=5).mask_type is AttentionMaskType.SLIDING_WINDOW
    assert FlashAttentionConfig(sliding_window=5).window_size == 5
    assert FlashAttentionConfig(causal=False).mask_type is AttentionMaskType.FULL
    assert not FlashAttentionConfig(head_dim=64, num_heads=8).is_gqa
    with pytest.raises(ValueError):
        FlashAttentionConfig(num_heads=8, num_kv_heads=3)
    with pytest.raises(ValueError):
        FlashAttentionConfig().scale
    caps = BackendCapabilities(AttentionBackend.TCGEN05_FLASH)
    assert caps.has_flex_attention and caps.has_flash_attention_2 and not caps.has_triton
    f = FlexAttentionConfig(num_attention_heads=8, num_key_value_heads=4, head_dim=64)
    assert caps.select_optimal_backend(f) is AttentionBackend.TCGEN05_FLASH
    assert caps.select_optimal_backend(FlexAttentionConfig(head_dim=96)) is AttentionBackend.REFERENCE
    here = BackendCapabilities.detect()
    if not torch.cuda.is_available():
        assert here.cuda_capability is None and not here.supports_fp8 and not here.supports_bf16
        assert here.select_optimal_backend(f) is AttentionBackend.REFERENCE
    assert callable(here.flex_attention_fn) and callable(here.create_block_mask_fn)


def test_activation_memory_manager_named_storage():
    from trainscale_b200.parallel.pipeline import ActivationMemoryManager
    m = ActivationMemoryManager()
    a, b = torch.ones(4, 4), torch.zeros(2)
    m.store_activation(0, "x", a)
    m.store_activation(0, "y", b)
    m.store_activation(1, "x", b)
    assert m.retrieve_activation(0, "x") is a and m.retrieve_activation(5, "x") is None
    assert m.current_memory_mb == pytest.approx((64 + 8 + 8) / 2 ** 20)
    assert m.release_activation(0) == 2 and m.retrieve_activation(0, "x") is None
    assert m.retrieve_activation(1, "x") is b and m.current_memory_mb == pytest.approx(8 / 2 ** 20)


def test_base_optimizer_grad_scale_step_count_and_close():
    from trainscale_b200.optim import BaseOptimizer, OptimizerState

    class SGD(BaseOptimizer):
        def __init__(self, params, lr=0.1):
            super().__init__(params, {"lr": lr})
        def _update(self, p, grad, state, group):
            p.add_(grad, alpha=-group["lr"])

    w = nn.Parameter(torch.ones(3))
    o = SGD([w])
    w.grad = torch.full((3,), 4.0)
    o.set_grad_scale(4.0)                                  # the loss was scaled by 4: the true gradient is 1
    o.step()
    assert torch.allclose(w.data, torch.full((3,), 0.9)) and o.step_count == 1 and o.get_grad_scale() == 4.0
    assert o.get_metrics() is o.metrics
    w.grad = torch.full((3,), 10.0)
    before = o.clip_grad_norm_(1.0)
    assert float(before) == pytest.approx(300 ** 0.5) and float(w.grad.norm()) == pytest.approx(1.0, abs=1e-5)
    o.close()
    assert o.lifecycle is OptimizerState.CLOSED and len(o.state) == 0
    with pytest.raises(RuntimeError):
        o.step()
    with pytest.raises(ValueError):
        o.set_grad_scale(0.0)


def test_adafactor_footprint_and_state_round_trip():
    from trainscale_b200.optim import AdaFactor, AdaFactorState
    w, b = nn.Parameter(torch.randn(8, 4)), nn.Parameter(torch.randn(4))
    o = AdaFactor([w, b])
    w.grad, b.grad = torch.randn(8, 4), torch.randn(4)
    o.step()
    fp = o.memory_footprint()
    assert fp["state_bytes"] == (8 + 4 + 4) * 4 and fp["total_bytes"] == fp["state_bytes"] + fp["buffer_bytes"]
    ps = o.profiling_stats
    assert ps.num_factorized_params == 1 and ps.num_full_params == 1 and ps.total_step_time_ns > 0
    s = AdaFactorState((8, 4), "cpu", torch.float32, True, True).initialize()
    s.step = 3
    s.exp_avg.fill_(2.0)
    back = AdaFactorState.from_dict(s.to_dict())
    assert back.step == 3 and back.factored and back.is_initialized and torch.equal(back.exp_avg, s.exp_avg)
    assert back.exp_avg is not s.exp_avg and back.memory_footprint() == s.memory_bytes() == (8 * 4 + 8 + 4) * 4


def test_cp_balancers_stateless_forms_and_ring_step():
    from trainscale_b200.parallel.cp import (BalancerStrategy, HeadTailBalancer, PTRRBalancer, RingCommunicator,
                                             ZigZagBalancer)
    x = torch.arange(32).view(1, 32)
    for cls in (HeadTailBalancer, ZigZagBalancer, PTRRBalancer):
        b = cls(4, 0)
        parts = [b.partition(x, r, 4, 1) for r in range(4)]
        assert torch.equal(b.gather(parts, 4, 1), x)
        for r in range(4):                                  # global positions ARE the values of arange at those places
            assert torch.equal(b.compute_global_positions(8, r, 4, 32), parts[r][0])
        with pytest.raises(ValueError):
            b.compute_global_positions(7, 0, 4, 32)
    assert HeadTailBalancer(4, 0).compute_global_positions(8, 1, 4).tolist() == [4, 5, 6, 7, 24, 25, 26, 27]
    st = BalancerStrategy("zigzag")
    assert torch.equal(st.gather([st.partition(x, r, 4, 1) for r in range(4)], 4, 1), x)
    assert st.compute_global_positions(8, 1, 4, 32).tolist() == [1, 6, 9, 14, 17, 22, 25, 30]
    ring = RingCommunicator()
    k, v = torch.randn(2, 3), torch.randn(2, 3)
    with ring.ring_step_context(k, v) as (kn, vn):
        pass
    assert torch.equal(kn, k) and torch.equal(vn, v)        # a ring of one rank hands back its own blocks


def test_fp8_scale_manager_and_linear_members():
    from trainscale_b200.kernels import FP8Config, FP8Linear, FP8ScaleManager
    lin = nn.Linear(256, 128)
    m = FP8Linear.from_linear(lin)
    x = torch.randn(4, 256)
    assert torch.allclose(m(x), lin(x), atol=1e-4) and (m.in_features, m.out_features) == (256, 128)
    q, sc = m.quantize_weight(lin.weight.data)
    assert q.dtype == torch.float8_e4m3fn and tuple(sc.shape) == (1, 2)
    with pytest.raises(ValueError):
        m.quantize_weight(torch.zeros(3, 3))
    mgr = FP8ScaleManager(FP8Config(amax_history_len=4))
    s, si = mgr.update_and_get_scale(torch.tensor([1.0, -2.0]), "act")
    assert float(s) == pytest.approx(2 / 448) and float(si) == pytest.approx(224.0)
    mgr.step()
    s, _ = mgr.update_and_get_scale(torch.tensor([0.5]), "act")
    assert float(s) == pytest.approx(2 / 448)                # the history still holds the earlier amax of 2
    assert mgr.get_meta("act") is mgr.get_meta("act")
    assert FP8Config().forward_spec.max_val == 448.0 and FP8Config().backward_spec.max_val == 57344.0


def test_function_classes_expose_forward_backward_pair():
    import types
    from trainscale_b200.kernels import FusedRoPEQKFunction, RMSLayerNormFunction, RoPEConfig, RoPEFrequencyCache
    x, w = torch.randn(2, 5, 16), torch.randn(16)
    ctx = types.SimpleNamespace()
    y = RMSLayerNormFunction.forward(ctx, x, w, 1e-6, True)
    gx, gw, g_eps, g_flag = RMSLayerNormFunction.backward(ctx, torch.ones_like(y))
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    RMSLayerNormFunction.apply(xr, wr, 1e-6, True).sum().backward()
    assert torch.allclose(gx, xr.grad) and torch.allclose(gw, wr.grad) and g_eps is None and g_flag is None

    class Mine(torch.autograd.Function):
        @staticmethod
        def forward(ctx, a, b):
            return RMSLayerNormFunction.forward(ctx, a, b)
        @staticmethod
        def backward(ctx, g):
            return RMSLayerNormFunction.backward(ctx, g)

    x2 = x.clone().requires_grad_(True)
    Mine.apply(x2, w).sum().backward()
    assert torch.allclose(x2.grad, xr.grad)
    cos, sin = RoPEFrequencyCache.get_freqs(RoPEConfig(dim=8), 5, "cpu", torch.float32)
    assert cos.shape == (5, 4)
    q, k = torch.randn(1, 5, 2, 8), torch.randn(1, 5, 2, 8)
    ctx = types.SimpleNamespace()
    q2, k2 = FusedRoPEQKFunction.forward(ctx, q, k, cos, sin)
    grads = FusedRoPEQKFunction.backward(ctx, torch.ones_like(q2), torch.ones_like(k2))
    assert grads[0].shape == q.shape and grads[1].shape == k.shape
    # rotation preserves norms, and so does its transpose applied to the gradient
    assert torch.allclose(q2.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    RoPEFrequencyCache.clear_cache()
    assert len(RoPEFrequencyCache._shared._cache) == 0


def test_distributed_metric_buffer_local_views():
    from trainscale_b200.metrics import DistributedMetricBuffer
    b = DistributedMetricBuffer()
    b.add("loss", 1.0)
    b.add("loss", torch.tensor(3.0))
    b.add("acc", 0.5)
    assert b.counts() == {"loss": 2, "acc": 1} and b.local_sums() == {"loss": 4.0, "acc": 0.5}
    assert b.local_means() == {"loss": 2.0, "acc": 0.5} and b.reduce_all() == {"loss": 2.0, "acc": 0.5}
    s = DistributedMetricBuffer("sum")
    s.add("tokens", 5)
    s.add("tokens", 7)
    assert s.reduce_all() == {"tokens": 12.0}
    b.clear()
    assert b.counts() == {} and b.reduce_all() == {}
    with pytest.raises(ValueError):
        DistributedMetricBuffer("max")


def test_hub_policy_members_and_result_map_err(tmp_path):
    from trainscale_b200.core.errors import HubError
    from trainscale_b200.core.types import Err, Ok
    from trainscale_b200.hub import CheckpointManager, CircuitBreaker, HubErrorCode, HubMetrics, RetryPolicy
    assert HubError("x", code=HubErrorCode.TIMEOUT).is_retriable
    assert not HubError("x", code=HubErrorCode.VALIDATION_ERROR).is_retriable and not HubError("y").is_retriable
    assert Ok(1).map_err(str) == Ok(1) and Err(2).map_err(lambda e: e * 2) == Err(4)
    now = [0.0]
    cb = CircuitBreaker(1, 10.0, clock=lambda: now[0])
    assert cb.can_execute().is_ok()
    cb.record_failure()
    r = cb.can_execute()
    assert r.is_err() and r.error.code is HubErrorCode.CIRCUIT_OPEN and r.error.context["retry_after_s"] == 10.0
    now[0] = 11.0
    assert cb.can_execute().is_ok()                          # half-open: one trial request may pass
    assert RetryPolicy(jitter=0).compute_delay_ms(2) == 2000
    m = HubMetrics()
    m.record_upload(10, 5_000_000, True)
    m.record_upload(10, 9_000_000, False)
    assert m.get_percentile_latency_ns(50) == 9_000_000 and m.get_percentile_latency_ns(50, "download") is None
    snap = m.snapshot()
    assert snap["uploads"] == {"total": 2, "failed": 1, "bytes": 10, "p50_latency_ms": 9.0, "p99_latency_ms": 9.0}
    cm = CheckpointManager(tmp_path)
    for step, loss in ((1, 2.0), (2, 1.0), (3, 1.5)):
        cm.save(step, lambda p: None, {"eval_loss": loss})
    assert cm.get_latest_checkpoint().step == 3
    best = cm.get_best_checkpoint()
    assert best.step == 2 and best.loss == 1.0
    assert CheckpointManager(tmp_path / "empty").get_best_checkpoint() is None


def test_grpo_compute_log_probs_match_full_logits():
    from trainscale_b200.models.llama import build_model
    from trainscale_b200.rl import GRPOCompute
    torch.manual_seed(0)
    m = build_model("tiny", dtype=torch.float32, device="cpu")
    g = GRPOCompute(group_size=2, model=m, reward_clip=0.8)
    ids = torch.randint(0, 1000, (4, 9))
    mask = torch.ones_like(ids)
    mask[0, 6:] = 0
    lp = g.compute_log_probs(ids, mask)
    with torch.no_grad():
        ref = torch.log_softmax(m(input_ids=ids).logits.float(), -1)[:, :-1].gather(-1, ids[:, 1:, None]).squeeze(-1)
    assert lp.shape == (4, 8) and torch.allclose(lp[1:], ref[1:], atol=1e-4)
    assert torch.allclose(lp[0, :5], ref[0, :5], atol=1e-4) and float(lp[0, 5:].abs().sum()) == 0.0   # padding targets
    loss, stats = g.compute_grpo_loss(lp, ref - 0.1, torch.tensor([1.0, 0.0, 0.5, 0.2]), mask[:, 1:].float())
    loss.backward()
    assert stats["reward_mean"] == pytest.approx(0.375) and stats["kl"] > 0      # the reward of 1.0 was clipped to 0.8
    assert m.head_weight.grad is not None


def test_small_members_of_configs_and_records():
    from trainscale_b200.callbacks import HOOKS, Callback
    from trainscale_b200.config.data_schema import DatasetConfig, PromptTemplate, SplitSpec, StageConfig
    from trainscale_b200.config.sota_config import SchedulerConfig
    from trainscale_b200.data.dataset_wrappers import StreamingPreprocessedDataset
    from trainscale_b200.data.length_manager import TokenAwareContentDistributor
    from trainscale_b200.inference.engine import GenerationParams, InferenceRequest, MetricsAggregator, RequestMetrics
    from trainscale_b200.introspection import ColumnMapper, DatasetIntrospector
    from trainscale_b200.kernels import FlexAttentionConfig
    from trainscale_b200.losses import CLIPLoss, LossRegistry
    from trainscale_b200.optim import KahanAccumulator, Prodigy
    from trainscale_b200.parallel.activation import CheckpointSegment, OffloadHandle, OffloadTarget
    from trainscale_b200.parallel.cp import BalancedCPScheduler, HybridCPConfig
    from trainscale_b200.parallel.ddp import DDPConfig, GradientCompression, GradientCompressionHook
    from trainscale_b200.parallel.dist_kernels import CommStreamManager, DistributedBackend, DistributedConfig
    from trainscale_b200.parallel.dist_utils import GradientSynchronizer, HardwareTopology
    from trainscale_b200.parallel.fsdp2 import ComputeCapability
    from trainscale_b200.parallel.mesh import (CommAlgorithmSelector, CommunicationAlgorithm, InterconnectType,
                                               MemoryEstimator)
    from trainscale_b200.trainer.sota_trainer import TrainingState

    st = TrainingState(global_step=3)
    st2 = st.with_update(global_step=4, epoch=1)
    assert (st.global_step, st2.global_step, st2.epoch) == (3, 4, 1)
    assert TokenAwareContentDistributor(max_length=100, special_tokens_budget=10).available_tokens == 90
    assert SchedulerConfig(warmup_steps=0, warmup_ratio=0.1).compute_warmup_steps(1000) == 100
    assert SchedulerConfig(warmup_steps=7).compute_warmup_steps(1000) == 7
    d = GenerationParams(max_tokens=5, top_k=0, seed=3, stop=["x"]).to_sampling_params()
    assert d["top_k"] == -1 and d["seed"] == 3 and d["stop"] == ["x"] and "logprobs" not in d
    with pytest.raises(ValueError):
        GenerationParams(n=0).to_sampling_params()
    assert InferenceRequest("p", lora_name="a", lora_path="/x", lora_id=2).get_lora_request()["lora_int_id"] == 2
    assert InferenceRequest("p", lora_name="a").get_lora_request() is None
    agg = MetricsAggregator()
    assert agg.summarize() == {"status": "no_requests_completed"}
    agg.record(RequestMetrics("r", 3, 4))
    assert agg.summarize()["requests"] == 1
    md = DatasetIntrospector().discover({"train": [{"question": "q", "answer": "a"}], "test": []}).unwrap()
    assert md.get_all_splits() == ["train", "test"] and md.get_config("default").splits[0].num_examples == 1
    assert md.get_config("nope") is None and md.get_all_splits("nope") == []
    sug = {m.target: m.source for m in ColumnMapper().suggest_mappings(["question", "answer", "id"])}
    assert sug == {"prompt": "question", "completion": "answer"}
    ds = DatasetConfig("d", stages={"s1": StageConfig("s1", {"train": SplitSpec("train")})})
    assert ds.is_staged() and ds.get_split_spec("train", "s1").name == "train" and ds.get_split_spec("train") is None
    assert not DatasetConfig("d").is_staged()
    assert PromptTemplate(input_columns=("a", "b"), label_column="b").get_required_columns() == ["a", "b"]
    assert PromptTemplate(input_columns=("a",), label_column="y").get_required_columns() == ["a", "y"]
    assert FlexAttentionConfig(num_attention_heads=8, num_key_value_heads=2, head_dim=64).kv_hidden_size == 128
    assert float(CLIPLoss(0.07).temperature) == pytest.approx(0.07, rel=1e-5)
    assert type(LossRegistry.get("focal")).__name__ == "FocalLoss" and "dpo" in LossRegistry.list_available()
    k = KahanAccumulator()
    k.add(1.0)
    k.reset()
    assert k.value == 0.0
    assert Prodigy([nn.Parameter(torch.zeros(2))], d0=1e-5).d == 1e-5
    assert OffloadHandle(0, (2, 3), torch.bfloat16, torch.device("cpu"), OffloadTarget.GPU).memory_bytes == 12
    assert CheckpointSegment(0, 2, 7).num_layers == 5
    assert MemoryEstimator.check_memory_fit(100, 80).is_ok() and MemoryEstimator.check_memory_fit(100, 95).is_err()
    assert "on_load" in HOOKS and Callback().on_load(None) is None
    assert ComputeCapability(10, 0).supports_flash_attention_v2 and not ComputeCapability(7, 5).supports_flash_attention_v2
    assert DistributedBackend.NCCL.to_torch_backend() == "nccl" and DistributedBackend.NONE.to_torch_backend() is None
    DistributedConfig(tp_size=2, pp_size=2, dp_size=2).validate_topology(8)
    with pytest.raises(ValueError):
        DistributedConfig(tp_size=2).validate_topology(8)
    assert DDPConfig.from_dict({"gradient_compression": "POWERSGD", "powersgd_rank": 8}).unwrap().gradient_compression \
        is GradientCompression.POWERSGD
    assert DDPConfig.from_dict({"no_such_option": 1}).is_err()
    hook = GradientCompressionHook()
    hook(None, torch.ones(8))
    assert hook.metrics.bytes_reduced == 32 and hook.metrics.compression_ratio == 1.0
    sel = CommAlgorithmSelector
    assert sel.select_allreduce_algorithm(1 << 10, 8, None, True) is CommunicationAlgorithm.NCCL_AUTO
    assert sel.select_allreduce_algorithm(1 << 10, 8) is CommunicationAlgorithm.TREE
    assert sel.select_allreduce_algorithm(1 << 26, 8) is CommunicationAlgorithm.RING
    env = sel.get_nccl_env_vars(CommunicationAlgorithm.RING, InterconnectType.NVLINK5)
    assert env == {"NCCL_P2P_LEVEL": "NVL", "NCCL_ALGO": "Ring"}
    assert sel.get_nccl_env_vars(CommunicationAlgorithm.NCCL_AUTO) == {}
    topo = HardwareTopology(2, "x", 1.0, 1, ((True, True), (True, True)))
    assert topo.total_gpus == 2 and topo.has_nvlink and not HardwareTopology(1, "x", 1.0, 1, ((True,),)).has_nvlink
    mgr = CommStreamManager(device="cpu")
    assert mgr.record_compute_event() is None and mgr.sync_back_to_compute() is None
    lin = nn.Linear(2, 2)
    lin(torch.ones(1, 2)).sum().backward()
    GradientSynchronizer(lin).sync_gradients()                # single process: gradients stay as they are
    assert lin.weight.grad is not None

    sched = BalancedCPScheduler(HybridCPConfig(max_tokens_per_rank=100, world_size=4))
    groups, ids = sched.get_groups_and_subsamples([(10, 400), (11, 90), (12, 100), (13, 180), (14, 50)])
    assert sorted(i for g in ids for gpu in g for i in gpu if True) .count(10) == 4      # 400 tokens: all four GPUs
    assert {i for g in ids for gpu in g for i in gpu} == {10, 11, 12, 13, 14}
    assert all(len(g) == 4 for g in groups) and groups[0][0][0] == (10, 4)

    class Ex:
        def __init__(self, row):
            self.row = row
        def to_dict(self):
            return {"input_ids": [self.row["v"]]}

    class Engine:
        def process(self, row):
            return Ex(row)

    stream = StreamingPreprocessedDataset([{"v": i} for i in range(50)], Engine())
    a = [int(x["input_ids"][0]) for x in stream.shuffle(buffer_size=8, seed=1)]
    b = [int(x["input_ids"][0]) for x in stream.shuffle(buffer_size=8, seed=1)]
    assert sorted(a) == list(range(50)) and a != list(range(50)) and a == b


def test_seq2seq_trainer_greedy_generate():
    from trainscale_b200.config.training_args import TrainingArguments
    from trainscale_b200.trainer.base import PretrainingTrainer, Seq2SeqTrainer

    class Toy(nn.Module):
        """Next decoder token = previous token + 1 (mod 6), whatever the encoder input."""
        def __init__(self):
            super().__init__()
            self.p = nn.Parameter(torch.zeros(1))
        def forward(self, input_ids, decoder_input_ids, **kw):
            nxt = (decoder_input_ids + 1) % 6
            return (torch.nn.functional.one_hot(nxt, 6).float() + self.p,)

    t = Seq2SeqTrainer(Toy(), TrainingArguments())
    out = t.generate({"input_ids": torch.zeros(2, 3, dtype=torch.long)}, max_length=8, eos_token_id=4)
    assert out.tolist() == [[1, 2, 3, 4]] * 2                 # stops once every row has produced the end token
    out = t.generate({"input_ids": torch.zeros(1, 3, dtype=torch.long)}, max_length=4)
    assert out.tolist() == [[1, 2, 3, 4]]
    pt = PretrainingTrainer(Toy(), TrainingArguments(), ema_decay=0.9)
    assert pt.ema_model is pt.ema and pt.ema_model is not pt.model
