"""Functions that share a name with the reference also take the reference's way of calling them: its keyword
spellings, its positional orders where they differ, its tensor layouts and return conventions."""
import os

import pytest
import torch
import torch.nn as nn


def test_reference_kwargs_decorator():
    import inspect

    from trainscale_b200.utils.refargs import ANY, reference_kwargs

    @reference_kwargs({"async_op": (False, None), "hint": ANY}, input_="x")
    def f(x, k=1):
        return x * k

    assert f(2) == 2 and f(input_=3, k=2) == 6 and f(x=1, async_op=False, hint="anything") == 1
    assert list(inspect.signature(f).parameters) == ["x", "k", "input_", "async_op", "hint"]
    with pytest.raises(NotImplementedError):
        f(1, async_op=True)                        # a request this framework does not honour is refused, not dropped
    with pytest.raises(TypeError):
        f(x=1, input_=2)


def test_result_helpers_and_small_renames():
    from trainscale_b200.core.types import Err, Ok, is_ok, map_result, unwrap_or
    from trainscale_b200.data.collate import pad_sequence_right
    from trainscale_b200.data.packing import get_packing_stats, pack_sequences, unpack_sequences
    from trainscale_b200.introspection import levenshtein_distance
    from trainscale_b200.metrics import sync_metric, sync_metrics
    assert is_ok(result=Ok(1)) and map_result(result=Ok(1), f=lambda v: v + 1) == Ok(2) and unwrap_or(result=Err(1), default=5) == 5
    assert levenshtein_distance(s1="ab", s2="b") == 1
    assert get_packing_stats([3, 4], max_seq_len=8)["num_packed"] == 1
    assert sync_metric(1.0, operation="mean", process_group=None) == 1.0 and sync_metrics(metrics={"a": 1.0}, operation="sum") == {"a": 1.0}
    assert pad_sequence_right(sequences=[torch.ones(2), torch.ones(3)], padding_value=0).shape == (2, 3)
    packed = pack_sequences(input_ids=[[1, 2, 3], [4, 5]], attention_mask=[[1, 1, 1], [1, 1]], labels=[[1, 2, 3], [4, 5]],
                            max_seq_len=8, pad_token_id=0, label_pad_id=-100)
    assert packed[0]["input_ids"].tolist() == [1, 2, 3, 4, 5, 0, 0, 0]
    parts = unpack_sequences(packed_output=torch.arange(5), cu_seqlens=torch.tensor([0, 3, 5]), original_lengths=[2, 2])
    assert [p.tolist() for p in parts] == [[0, 1], [3, 4]]


def test_attention_functions_in_the_reference_layout():
    from trainscale_b200 import kernels as K
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 5, 4, 8), torch.randn(2, 5, 2, 8), torch.randn(2, 5, 2, 8)
    t = lambda x: x.transpose(1, 2)        # noqa: E731  [B, S, H, D] <-> [B, H, S, D]
    ours = K.flash_attention(q, k, v)
    theirs = K.flash_attention(query=t(q), key=t(k), value=t(v), causal=True)
    assert torch.allclose(ours, t(theirs), atol=1e-6)
    full = K.flash_attention(query=t(q), key=t(k), value=t(v))               # the reference's default is NOT causal
    assert not torch.allclose(full, theirs, atol=1e-3)
    assert K.flash_attention(query=t(q), key=t(k), value=t(v), return_softmax=True).output.shape == (2, 4, 5, 8)
    with pytest.raises(NotImplementedError):
        K.flash_attention(query=t(q), key=t(k), value=t(v), dropout_p=0.1)
    assert torch.allclose(K.naive_attention(q, k, v), t(K.naive_attention(query=t(q), key=t(k), value=t(v), causal=True)), atol=1e-6)
    cfg = K.FlexAttentionConfig(attn_logit_softcapping=30.0, query_pre_attn_scalar=8)
    a = K.slow_attention_softcapping(q, k, v, 30.0)
    b = K.slow_attention_softcapping(Q=t(q), K=t(k), V=t(v), causal_mask=object(), config=cfg)
    assert torch.allclose(a.reshape(2, 5, -1), b, atol=1e-6)
    c = K.attention_softcapping_compiled(Q=t(q), K=t(k), V=t(v), causal_mask=1, query_scalar=8, softcap=30.0,
                                         num_heads=4, num_kv_heads=2, head_dim=8)
    assert torch.allclose(b, c, atol=1e-5)
    Qd, Kd, Vd = torch.randn(2, 4, 1, 8), torch.randn(2, 2, 6, 8), torch.randn(2, 2, 6, 8)
    o = K.inference_attention_single_token(Q=Qd, K=Kd, V=Vd, config=None)
    ref = torch.nn.functional.scaled_dot_product_attention(Qd, Kd.repeat_interleave(2, 1), Vd.repeat_interleave(2, 1))
    assert torch.allclose(o, ref.transpose(1, 2).reshape(2, 1, -1), atol=1e-5)
    assert K.create_causal_mask(max_seq_len=3).shape == (3, 3)
    assert K.create_sliding_window_causal_mask(max_seq_len=4, window_size=2)[3, 1] == float("-inf")


def test_rope_lora_and_fp8_function_forms():
    from trainscale_b200 import kernels as K
    torch.manual_seed(0)
    cos, sin = K.precompute_freqs_cis(8, max_seq_len=16, dtype=torch.float32)
    Q, Kt = torch.randn(1, 5, 2, 8), torch.randn(1, 5, 1, 8)
    q2, k2 = K.apply_rope(Q, Kt, cos, sin)
    Qc, Kc = Q.clone(), Kt.clone()
    assert K.inplace_rope_embedding(Qc, Kc, cos, sin, 0)[0] is Qc and torch.allclose(Qc, q2) and torch.allclose(Kc, k2)
    assert torch.allclose(K.fast_rope_embedding(Q, cos, sin), q2)
    pair = K.fast_rope_embedding(Q, Kt, cos, sin)
    assert torch.allclose(pair[0], q2) and torch.allclose(pair[1], k2)

    x, W, A, B = torch.randn(4, 16), torch.randn(8, 16), torch.randn(2, 16), torch.randn(8, 2)
    want = x @ W.t() + 2.0 * (x @ A.t()) @ B.t()
    for got in (K.matmul_lora(x, W, A, B, 2.0), K.matmul_lora(x, W, None, A, B, 2.0), K.matmul_lora(x, W, A=A, B=B, scaling=2.0)):
        assert torch.allclose(got, want, atol=1e-4)
    with pytest.raises(NotImplementedError):
        K.matmul_lora(x, W, object(), A, B, 2.0)
    assert K.validate_lora_gradients(x, W, A, B, 2.0) is True and K.validate_lora_gradients()["passed"]

    class P(nn.Module):
        def __init__(self, o, i):
            super().__init__()
            self.weight, self.scaling = nn.Parameter(torch.randn(o, i)), 0.5
            self.lora_A, self.lora_B = nn.Parameter(torch.randn(2, i)), nn.Parameter(torch.randn(o, 2))
        def dense(self, h):
            return h @ self.weight.t() + 0.5 * (h @ self.lora_A.t()) @ self.lora_B.t()

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = P(32, 16), P(32, 16), P(16, 32)

    m = MLP()
    want = m.down_proj.dense(torch.nn.functional.silu(m.gate_proj.dense(x)) * m.up_proj.dense(x))
    assert torch.allclose(K.apply_lora_mlp_swiglu(m, x), want, atol=1e-4)
    assert torch.allclose(K.apply_lora_mlp_swiglu(mlp_module=m, X=x, inplace=True), want, atol=1e-4)
    qp, kp, vp = P(8, 16), P(4, 16), P(4, 16)
    got = K.apply_lora_qkv(qp, kp, vp, x)
    assert all(torch.allclose(g, p.dense(x), atol=1e-4) for g, p in zip(got, (qp, kp, vp)))

    wq, ws = K.block_quantize_fp8(x=torch.randn(256, 256), block_size=128)
    assert wq.dtype == torch.float8_e4m3fn and ws.shape == (2, 2)
    wd = K.block_dequantize_fp8(y=wq, scales=ws, block_size=128, out_dtype=torch.float32)
    xq, xs = K.block_quantize_fp8(torch.randn(128, 256))
    out = K.fp8_matmul_block_scaled(A=xq, A_scale=xs, B=wq.t().contiguous(), B_scale=ws.t().contiguous(), out_dtype=torch.float32)
    assert torch.allclose(out, K.block_dequantize_fp8(xq, xs, 128, torch.float32) @ wd.t(), atol=1e-3)
    Aq, As = K.row_quantize_fp8(x=torch.randn(8, 32))
    Bq, Bs = K.row_quantize_fp8(torch.randn(16, 32))
    out = K.fp8_matmul_row_scaled(Aq, As, Bq.t(), Bs, out_dtype=torch.float32)
    assert torch.allclose(out, (Aq.float() * As) @ (Bq.float() * Bs).t(), atol=1e-4)
    assert K.row_quantize_fp8(torch.randn(2, 8), fp8_format="e5m2")[0].dtype == torch.float8_e5m2

    z, y = torch.randn(4, 7), torch.tensor([1, 2, 3, -100])
    capped = 30.0 * torch.tanh(z / 30.0)
    want = torch.nn.functional.cross_entropy(capped, y, ignore_index=-100, reduction="sum") / 3
    assert torch.allclose(K.fast_cross_entropy_loss(z, y, logit_softcapping=30.0, n_items=3), want, atol=1e-5)
    assert K.fused_add_rms_layernorm(X=torch.randn(2, 8), residual=torch.randn(2, 8), weight=torch.ones(8)).shape == (2, 8)
    assert len(K.fused_add_rms_layernorm(torch.randn(2, 8), torch.randn(2, 8), torch.ones(8), return_residual=True)) == 2
    assert torch.allclose(K.fused_gelu(torch.ones(2), approx=True), torch.nn.functional.gelu(torch.ones(2), approximate="tanh"))


def test_rl_functions_reference_forms():
    from trainscale_b200.rl import (chunked_log_softmax, compute_advantages, dapo_loss, drgrpo_loss, grpo_loss,
                                    left_pack_padding, selective_log_softmax)
    torch.manual_seed(0)
    B, G, L = 2, 3, 4
    p, r = torch.randn(B, G, L, requires_grad=True), torch.randn(B, G, L)
    m, rew = torch.ones(B, G, L), torch.randn(B, G)
    adv = compute_advantages(rew, baseline="mean")
    assert adv.shape == (B, G) and torch.allclose(adv.mean(-1), torch.zeros(B), atol=1e-6)
    assert torch.allclose(compute_advantages(rew, "none"), rew / rew.std())
    lp = (p * m).sum(-1) / m.sum(-1)
    loss, met = grpo_loss(policy_log_probs=p, ref_log_probs=r, advantages=adv, mask=m, beta=0.04)
    want = -(adv * lp).mean() + 0.04 * ((p - r) * m).sum(-1).mean() / m.sum(-1).mean()
    assert torch.allclose(loss, want, atol=1e-6) and set(met) == {"pg_loss", "kl_loss", "kl_div", "total_loss"}
    loss, met = drgrpo_loss(policy_log_probs=p, ref_log_probs=r, advantages=adv, mask=m, epsilon=0.1)
    assert "ratio_mean" in met and loss.requires_grad
    loss, met = dapo_loss(policy_log_probs=p, ref_log_probs=r, rewards=rew, mask=m, temperature=2.0)
    soft = torch.softmax(rew / 2.0, -1)
    assert torch.allclose(loss, -(soft * lp).sum(-1).mean() + 0.04 * (((p - r) * m).sum(-1) / m.sum(-1)).mean(), atol=1e-6)
    # this framework's positional forms are unchanged
    flat = torch.randn(6, L)
    assert grpo_loss(flat, flat.detach(), None, compute_advantages(torch.randn(6), 3), torch.ones(6, L)).dim() == 0

    ids = torch.tensor([[5, 6, 0, 0], [7, 0, 0, 0]])
    assert left_pack_padding(ids, 0).tolist() == [[0, 0, 5, 6], [0, 0, 0, 7]]            # the reference's direction
    assert left_pack_padding(input_ids=ids, pad_token_id=0).tolist() == [[0, 0, 5, 6], [0, 0, 0, 7]]
    packed, mask = left_pack_padding(torch.tensor([[0, 5, 0, 6]]), torch.tensor([[0, 1, 0, 1]]))
    assert packed.tolist() == [[5, 6, 0, 0]] and mask.tolist() == [[1, 1, 0, 0]]

    lg, idx = torch.randn(2, 3, 7), torch.randint(0, 7, (2, 3))
    want = torch.log_softmax(5.0 * torch.tanh(lg / 5.0) / 2.0, -1).gather(-1, idx[..., None]).squeeze(-1)
    assert torch.allclose(selective_log_softmax(lg, input_ids=idx, temperature=2.0, logit_softcapping=5.0), want, atol=1e-5)
    h, W = torch.randn(2, 3, 8), torch.randn(7, 8)
    got = chunked_log_softmax(hidden_states=h, lm_head=W, input_ids=idx, num_chunks=2, temperature=2.0)
    assert torch.allclose(got, selective_log_softmax(h @ W.t(), idx, 2.0), atol=1e-4)
    got = chunked_log_softmax(h, W, idx, num_chunks=2, logit_softcapping=5.0)
    assert torch.allclose(got, selective_log_softmax(h @ W.t(), idx, 1.0, 5.0), atol=1e-4)


def test_config_export_quantization_forms(tmp_path):
    from trainscale_b200.config.sota_config import get_dpo_preset, get_qlora_preset
    from trainscale_b200.config.training_args import load_training_config, merge_configs
    from trainscale_b200.export import create_vllm_config, push_to_hub, save_safetensors
    from trainscale_b200.hub import generate_model_card
    from trainscale_b200.quantization import (QuantizationConfig, estimate_memory_usage, fast_dequantize,
                                              quantize_nf4_param)
    assert get_qlora_preset(model_name="x", max_seq_length=512).data.max_seq_length == 512
    assert get_dpo_preset("y").model.name_or_path == "y" and merge_configs({"a": 1}, overrides={"a": 2}) == {"a": 2}
    f = tmp_path / "t.yaml"
    f.write_text("section:\n  learning_rate: 0.5\n  output_dir: ${TS_TEST_UNSET:-out}\n")
    cfg = load_training_config(yaml_path=f, config_key="section")
    assert cfg.learning_rate == 0.5 and cfg.output_dir == "out"
    assert load_training_config(f, config_key="section", interpolate_env=False).output_dir.startswith("${")
    m = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4))
    out = save_safetensors(m, output_dir=tmp_path / "w", max_shard_size="1MB")
    assert (out / "model.safetensors").exists()
    assert create_vllm_config(str(out), str(tmp_path / "serve")).parent == tmp_path / "serve"
    assert push_to_hub(m, None, "someone/model") is None                       # offline: nothing is uploaded
    card = generate_model_card(m, "my-model", description="d", license="mit", language="en")
    assert "# my-model" in card and "license: mit" in card and "Parameters" in card
    est = estimate_memory_usage(7.0, QuantizationConfig(load_in_4bit=True))
    assert est["model_gb"] == pytest.approx(7e9 * 0.5 / 2 ** 30, abs=0.01) and est["gradient_gb"] == est["lora_gb"]
    assert "weights_gb" in estimate_memory_usage(7e9)
    assert fast_dequantize(torch.ones(2), None, torch.float32).dtype == torch.float32
    w = torch.randn(8, 64)
    assert (fast_dequantize(quantize_nf4_param(w), out_dtype=torch.float32) - w).abs().max() < 0.5


def test_distributed_and_pipeline_function_forms(tmp_path):
    from trainscale_b200.parallel import tp as TP
    from trainscale_b200.parallel.activation import create_activation_checkpoint_from_config, print_offload_summary
    from trainscale_b200.parallel.cp import estimate_memory_per_gpu, hybrid_context_parallel_forward_backward
    from trainscale_b200.parallel.dist_utils import (dist_all_gather, dist_reduce, finalize_model_grads,
                                                     fused_clip_grad_norm_, load_checkpoint_distributed,
                                                     save_checkpoint_distributed, set_deterministic_seed)
    from trainscale_b200.parallel.pipeline import (PipelineConfig, ProfilingConfig, ScheduleType, balance_stages_by_memory,
                                                   create_schedule, estimate_stage_memory, merge_microbatches,
                                                   pipeline_profiler, selective_checkpoint, split_into_microbatches,
                                                   split_model_into_stages)
    m = nn.Linear(2, 2)
    m(torch.ones(1, 2)).sum().backward()
    finalize_model_grads([m], torch.tensor(4.0), sequence_parallel=False, qk_layernorm=False,
                         share_embeddings_and_output_weights=True)
    assert torch.allclose(m.weight.grad, torch.full((2, 2), 0.25))
    before = fused_clip_grad_norm_(model_or_params=m, max_norm=0.1, norm_type=2.0, process_group=None, foreach=True)
    assert float(before) == pytest.approx(6 ** 0.5 * 0.25, rel=1e-5)
    assert dist_reduce(tensor=torch.ones(1), op="sum", process_group=None, async_op=False).item() == 1.0
    assert len(dist_all_gather(tensor=torch.ones(1), contiguous=True)) == 1
    assert set_deterministic_seed(3, 5) == 8 and set_deterministic_seed(3, 5, per_rank_offset=False) == 3
    save_checkpoint_distributed({"a": torch.ones(2)}, tmp_path / "c.pt", None)
    assert load_checkpoint_distributed(tmp_path / "c.pt", None, "cpu")["a"].tolist() == [1.0, 1.0]

    x = torch.randn(2, 3)                                    # no registered group: the region functions are identities
    assert TP.copy_to_tensor_parallel_region(input_=x, async_op=False) is x
    assert TP.gather_from_tensor_parallel_region(x, dim=-1) is x
    with pytest.raises(NotImplementedError):
        TP.gather_from_tensor_parallel_region(x, dim=0)      # this function always gathers the last dimension
    lg, y = torch.randn(2, 3, 7), torch.randint(0, 7, (2, 3))
    got = TP.vocab_parallel_cross_entropy(logits=lg, targets=y, label_smoothing=0.1)
    want = torch.nn.functional.cross_entropy(lg.view(-1, 7), y.view(-1), label_smoothing=0.1, reduction="none").view(2, 3)
    assert torch.allclose(got, want, atol=1e-5)
    assert TP.shard_model_for_tensor_parallel(m, config=TP.TensorParallelConfig()) is m

    seq = nn.Sequential(*[nn.Linear(4, 4) for _ in range(6)])
    assert [len(s.module) for s in split_model_into_stages(seq, 3, balance=[1, 2, 3])] == [1, 2, 3]
    assert [len(s.module) for s in split_model_into_stages(seq, 2, split_points=["4"])] == [4, 2]
    with pytest.raises(ValueError):
        split_model_into_stages(seq, 3, balance=[1, 1, 1])
    mib = estimate_stage_memory([seq, seq], (2, 8), torch.float32)
    assert len(mib) == 2 and mib[0] == mib[1] > 0
    assert balance_stages_by_memory(model=seq, num_stages=2, input_shape=(2, 8), target_memory_mb=10) == [range(0, 3), range(3, 6)]
    stages = split_model_into_stages(seq, 3)
    sched = create_schedule(ScheduleType.GPIPE, stages, PipelineConfig(num_stages=3), nn.functional.mse_loss)
    assert type(sched).__name__ == "GPipeSchedule"
    assert type(create_schedule(stages, PipelineConfig(num_stages=3), nn.functional.mse_loss)).__name__ == "OneFOneBSchedule"
    assert len(split_into_microbatches(tensor=torch.ones(4, 2), num_microbatches=2)) == 2
    assert merge_microbatches(microbatches=[torch.ones(1, 2)] * 2).shape == (2, 2)
    xin = torch.ones(2, 4, requires_grad=True)
    selective_checkpoint(lambda a: a * 2, xin, preserve_rng_state=True).sum().backward()
    assert xin.grad[0, 0] == 2
    with pipeline_profiler(ProfilingConfig(enabled=False), str(tmp_path)) as prof:
        assert prof is None

    assert create_activation_checkpoint_from_config(config={"mode": "full"}).cfg.mode.value == "full"
    print_offload_summary({"attn": 2 ** 21, "mlp": 2 ** 20})
    one_layer = estimate_memory_per_gpu(batch_size=2, seq_len=8192, hidden_dim=4096, num_heads=32, cp_degree=4)
    assert isinstance(one_layer, int) and one_layer > 0
    assert estimate_memory_per_gpu(8192, 4, 4096, 32, 8, 128)["tokens_per_gpu"] == 2048

    lin = nn.Linear(2, 1)

    def forward_step(it, model):
        xb = next(it)
        out = model(xb)
        return out, lambda o: (o.pow(2).mean(), torch.tensor(xb.shape[0]), {"loss": float(o.pow(2).mean().detach())})

    store, tokens = hybrid_context_parallel_forward_backward(forward_step_func=forward_step, model=lin,
                                                             data_iterator=iter([torch.ones(3, 2)] * 4), num_microbatches=4)
    assert len(store) == 4 and int(tokens) == 12 and lin.weight.grad is not None


def test_data_and_serving_function_forms():
    from trainscale_b200.data.dataloader_factory import build_dataloader
    from trainscale_b200.data.length_manager import create_content_distributor, find_word_boundary
    from trainscale_b200.data.prompt_engine import render_template
    from trainscale_b200.inference.engine import EnginePresets, create_openai_server
    from trainscale_b200.registry import auto_patch_layernorm, get_model_info
    ds = [{"input_ids": torch.arange(n + 1), "labels": torch.arange(n + 1)} for n in range(4)]
    b = next(iter(build_dataloader(ds, batch_size=4, pad_token_id=9, label_pad_token_id=-1, padding_side="right")))
    assert b["input_ids"][0].tolist() == [0, 9, 9, 9] and b["labels"][0].tolist() == [0, -1, -1, -1]
    d = create_content_distributor(max_length=64, distribution_mode="proportional", column_ratios={"a": 0.5, "b": 0.5},
                                   default_truncation="right", chars_per_token=4.0)
    assert d.available_tokens == 54 and d.estimator.cpt == 4.0
    assert find_word_boundary("hello world foo", max_chars=8) == 6
    assert render_template("hi {x}", {"x": 1}, use_jinja=False) == "hi 1"
    assert get_model_info(model_id="meta-llama/x").family == "llama" and auto_patch_layernorm(module=nn.LayerNorm(4)) == 1
    cfg = EnginePresets.low_latency_interactive("tiny")
    cfg.device = "cpu"
    cfg.cache.num_gpu_blocks = 32
    app = create_openai_server(cfg, "127.0.0.1", port=8123)
    assert (app.state.host, app.state.port) == ("127.0.0.1", 8123)


def test_expert_parallel_blocks_take_the_reference_forms():
    """Routers return the dense routing record for `hidden_states=`; experts take activation / dropout / use_gated; the
    layers return (output, auxiliary loss, router logits); padded tokens are routed nowhere."""
    import warnings
    from trainscale_b200.parallel.ep import (AllToAllDispatcher, ExpertChoiceRouter, ExpertFFN, ExpertParallelConfig,
                                             ExpertParallelMoE, GroupedExperts, HierarchicalMoE, MoELayer, SoftMoERouter,
                                             TopKRouter)
    warnings.simplefilter("ignore")
    cfg = ExpertParallelConfig(num_experts=4, top_k=2, hidden_size=16, intermediate_size=32)
    torch.manual_seed(0)
    x = torch.randn(2, 5, 16)
    flat = x.reshape(-1, 16)
    pad = torch.zeros(2, 5, dtype=torch.bool)
    pad[1, 3:] = True
    out = TopKRouter(config=cfg)(hidden_states=x, padding_mask=pad)
    assert out.dispatch_mask.shape[:2] == (10, 4) and out.dispatch_mask[8:].sum() == 0
    assert abs(float(out.combine_weights.sum()) - 8.0) < 1e-4            # 8 live tokens, weights of a token sum to 1
    assert ExpertChoiceRouter(config=cfg)(hidden_states=x, padding_mask=pad).dispatch_mask[8:].sum() == 0
    soft = SoftMoERouter(config=cfg)(hidden_states=x, padding_mask=pad)
    assert torch.allclose(soft.dispatch_mask.sum(0), torch.ones(4, 1), atol=1e-5) and soft.dispatch_mask[8:].abs().sum() == 0
    plain = ExpertFFN(hidden_size=16, intermediate_size=32, activation="gelu", dropout=0.0, use_gated=False)
    assert plain.w_gate_up.shape == (32, 16)
    ref = torch.nn.functional.gelu(flat @ plain.w_gate_up.t()) @ plain.w_down.t()
    assert torch.allclose(plain(flat), ref, atol=1e-5)
    assert ExpertFFN(16, 32, "relu", 0.1, True)(x).shape == x.shape
    with pytest.raises(ValueError):
        ExpertFFN(16, 32, activation="nope")
    experts = GroupedExperts(4, hidden_size=16, intermediate_size=32)
    y = experts(tokens=flat, expert_indices=out.expert_indices, expert_weights=out.expert_weights)
    assert y.shape == flat.shape and y[8:].abs().sum() == 0              # padded tokens carry zero weights
    layer = MoELayer(config=cfg)
    o, aux, logits = layer(hidden_states=x, attention_mask=(~pad).long(), output_router_logits=True)
    assert o.shape == x.shape and logits.shape == (10, 4) and aux.dim() == 0 and o[1, 3:].abs().sum() == 0
    assert torch.allclose(layer(x)[0], o[0], atol=1e-6)
    ep = ExpertParallelMoE(config=cfg)                                    # no process group: every expert is local
    layer.load_state_dict(ep.state_dict())
    assert torch.allclose(ep(hidden_states=x)[0], layer(x), atol=1e-6) and ep.get_routing_statistics()["forward_count"] == 1
    ho, haux = HierarchicalMoE(config=cfg, num_groups=2)(hidden_states=x, attention_mask=(~pad).long())
    assert ho.shape == x.shape and ho[1, 3:].abs().sum() == 0 and haux.dim() == 0
    d = AllToAllDispatcher(4, 4, 6, None)
    mask = torch.zeros(10, 4, dtype=torch.bool).scatter_(1, out.expert_indices, True)
    rows, counts = d.dispatch(tokens=flat, dispatch_mask=mask)
    assert rows.shape == (4, 6, 16) and counts.tolist() == mask.sum(0).clamp(max=6).tolist()
    w = torch.zeros(10, 4).scatter_(1, out.expert_indices, out.expert_weights.detach())
    kept = (mask.long().cumsum(0) - 1 < 6) & mask
    back = d.combine(expert_outputs=rows, combine_weights=w, original_positions=torch.arange(10), num_tokens=10)
    assert torch.allclose(back, flat * (w * kept).sum(1, keepdim=True), atol=1e-5)


def test_context_parallel_classes_take_the_reference_forms():
    from trainscale_b200.parallel.cp import (BalancedCPScheduler, ContextParallel, ContextParallelAttention,
                                             ContextParallelConfig, ContextParallelEngine, RingBufferPool,
                                             RingCommunicator, TensorArena)

    class Group:
        def size(self):
            return 8

    s = BalancedCPScheduler(max_seq_len_per_rank=1024, dp_cp_group=Group())
    assert s.total_hdp_gpus == 8 and s.gpus_needed(seq_len=3000) == 4 and s.get_total_workload(seq_length=100, cp_size=2) == 5000.0
    samples = list(enumerate([4000, 3000, 900, 800, 700, 600, 500, 400, 300, 200, 100, 2048]))
    est = lambda l, cp=None: l * l / (cp or 1)                                   # noqa: E731
    buckets = s.make_buckets_equal(samples, est)
    assert len(buckets) == 3 and [x for b in buckets for x in b] == samples      # order kept, one bucket per CP degree
    micro, left, times, ids = s.next_hdp_group(samples, est, 8, delta=0.05, strategy="dp")
    assert len(micro) == len(times) == len(ids) == 8 and all(micro)             # no GPU idles
    assert micro[0] == [4000] and ids[0] == [0] and times[0] == 4000 * 4000 / 4
    placed = {i for gpu in ids for i in gpu}
    assert placed | {i for i, _ in left} == set(range(12)) and not placed & {i for i, _ in left}
    assert s.next_hdp_group([4000, 900, 800], 0) == ([(0, 4), (1, 1), (2, 1)], 3)            # the native form still works
    with pytest.raises(ValueError):
        s.next_hdp_group(samples, est, 8, strategy="zz")

    arena = TensorArena(capacity_bytes=1024, device="cpu", dtype=torch.float16)
    assert arena.size == 1024 and arena.default_dtype is torch.float16
    assert len(RingBufferPool((2, 3), torch.float32, "cpu", num_buffers=3, pin_memory=False).buffers) == 3
    assert len(RingBufferPool(2, (2, 3), torch.float32).buffers) == 2
    cfg = ContextParallelConfig(cp_degree=1)
    n = cfg.compute_memory_requirement(batch_size=2, seq_len=128, hidden_dim=64, num_heads=4)
    per = 2 * 128 * 64 * 2
    assert n == cfg.compute_memory_requirement(2, 128, 64, 4) == 3 * per + cfg.ring_buffer_count * 2 * per + per + 2 * 4 * 128 * 4
    assert isinstance(cfg.compute_memory_requirement(128, 64, 2, 4, 16), dict)
    ring = RingCommunicator(cp_rank=0, cp_world_size=1, process_group=None, device="cpu", k_shape=(1, 4, 2, 8),
                            v_shape=(1, 4, 2, 8), dtype=torch.float32)
    k, v = torch.randn(1, 4, 2, 8), torch.randn(1, 4, 2, 8)
    kr, vr, event = ring.start_send_recv(k_local=k, v_local=v)
    ring.wait_recv(event=event)
    assert torch.equal(kr, k) and torch.equal(vr, v)
    engine = ContextParallelEngine(cfg)
    assert engine.initialize(cp_mesh=None).is_ok()
    attn = ContextParallelAttention(cfg, engine, 16, 2)
    q = torch.randn(1, 6, 16)
    out = attn(q, q, q)
    heads_first = q.view(1, 6, 2, 8).transpose(1, 2)
    assert out.shape == q.shape
    assert torch.allclose(attn(heads_first, heads_first, heads_first).transpose(1, 2).reshape(1, 6, 16), out, atol=1e-6)
    wrapper = ContextParallel({"cp_degree": 1})
    ids_ = torch.arange(8).view(1, 8)
    shards = wrapper.shard_inputs(ids_, ids_.clone())
    assert len(shards) == 4 and shards[2] is None and torch.equal(shards[0], ids_)
    assert torch.equal(wrapper.restore_sequence(sharded_output=q, seq_dim=1), q)
    assert torch.equal(engine.gather_output(sharded_output=q), q)


def test_pipeline_and_checkpoint_classes_take_the_reference_forms():
    import torch.nn as nn
    from trainscale_b200.parallel.activation import (ActivationCheckpoint, ActivationCheckpointConfig, ActivationOffloader,
                                                     ActivationPool, SelectiveCheckpointPolicy)
    from trainscale_b200.parallel.dist_utils import TensorPool
    from trainscale_b200.parallel.pipeline import (ActivationMemoryManager, CheckpointFunction, CommunicationConfig,
                                                   GradientBucket, InterleavedOneFOneBSchedule, MemoryConfig,
                                                   P2PCommunicator, PipelineConfig, PipelineStage, VirtualPipelineStage)
    mem = ActivationMemoryManager(MemoryConfig(), "cpu")
    mem.stash_activation(0, 1, torch.ones(2))
    assert torch.equal(mem.pop_activation(0, 1), torch.ones(2))
    mem.stash_activation(stage_id=1, microbatch_id=2, activation=torch.zeros(1))
    assert mem.pop_activation(stage_id=1, microbatch_id=2).numel() == 1
    comm = P2PCommunicator(CommunicationConfig(), "cpu", None)
    assert comm.send_async(torch.ones(1), dst_rank=1, tag=0).is_err()           # no process group: an Err, not a raise
    assert comm.recv_sync(src_rank=0).is_err()
    bucket = GradientBucket(max_size_bytes=100, device="cpu", dtype=torch.float16)
    assert (bucket.capacity, bucket.dtype, bucket.device) == (100, torch.float16, "cpu")
    lin = nn.Linear(4, 4)
    x = torch.randn(2, 4, requires_grad=True)
    CheckpointFunction.apply(lambda a: lin(a).relu(), True, x).sum().backward()
    recomputed = lin.weight.grad.clone()
    lin.zero_grad()
    lin(x).relu().sum().backward()
    assert torch.allclose(recomputed, lin.weight.grad)
    config = PipelineConfig(num_stages=2, num_microbatches=2, memory=MemoryConfig(enable_activation_checkpointing=True))
    stage = PipelineStage(lin, 0, 2, None, config)
    assert stage.checkpoint_activations and stage(input_=x, checkpoint=True).shape == (2, 4)
    virtual = VirtualPipelineStage([stage, stage], virtual_stage_id=0, physical_stage_id=0)
    assert virtual.virtual_stage_id == 0 and virtual.forward(x, 1, True).shape == (2, 4) and virtual.forward(0, x).shape == (2, 4)
    native = VirtualPipelineStage([stage, stage], 1, 2)
    assert native.virtual_stage_id(1) == 3
    sched = InterleavedOneFOneBSchedule([PipelineStage(nn.Linear(4, 4), i, 4) for i in range(4)],
                                        PipelineConfig(num_stages=2, num_microbatches=2, schedule="interleaved"),
                                        lambda a, b: (a - b).pow(2).mean(), num_chunks=2)
    assert sched.num_chunks == 2 and sched.config.num_virtual_stages == 2
    model = nn.Sequential(lin)
    assert ActivationCheckpoint(config=ActivationCheckpointConfig()).apply(model, batch_size=2, seq_len=16) is model
    assert SelectiveCheckpointPolicy(config=ActivationCheckpointConfig()).config is not None
    assert ActivationOffloader(ActivationCheckpointConfig(), torch.device("cpu")).min_bytes == 1 << 20
    pool = ActivationPool(initial_capacity=2, max_capacity=1, device="cpu")
    pool.release(tensor=pool.acquire((2, 2), torch.float32))
    pool.release(tensor=torch.ones(3))                                         # over the buffer bound: not kept
    assert pool.get_stats()["buffers_cached"] == 1
    tensors = TensorPool("cpu", pin_memory=True)
    tensors.free(tensor=tensors.acquire((4,)))
    assert tensors.get_stats()["releases"] == 1


def test_zero_bubble_classes_take_the_reference_forms():
    import torch.nn as nn
    from trainscale_b200.parallel.pipeline import ActivationMemoryManager, MemoryConfig
    from trainscale_b200.parallel.zbpp import (GradientDecomposer, ModelPartitioner, PipelineStageModule, ScheduleConfig,
                                               SplitBackwardFunction, StageProfile, ZBPPBenchmark, ZBPPOptimizer,
                                               ZBPPRuntimeEngine, ZeroBubblePipeline)
    torch.manual_seed(0)
    decomposer = GradientDecomposer(False, torch.float32, True)
    memory = ActivationMemoryManager(MemoryConfig(), "cpu")
    x = torch.randn(6, 8, requires_grad=True)
    lin = nn.Linear(8, 4)
    y = SplitBackwardFunction.apply(x, lin.weight, lin.bias, 1, 3, decomposer, memory)
    go = torch.randn_like(y)
    y.backward(go)
    want = torch.autograd.grad(lin(x), [x, lin.weight, lin.bias], go)
    assert torch.allclose(x.grad, want[0], atol=1e-6) and torch.allclose(lin.bias.grad, want[2], atol=1e-6)
    assert lin.weight.grad is None                                             # the weight gradient is deferred ...
    deferred = decomposer.compute_b_params(memory.retrieve_activation(3, "stage_1_input"),
                                           memory.retrieve_activation(3, "stage_1_grad_output"), lin.weight)
    assert torch.allclose(deferred, want[1], atol=1e-5)                        # ... and comes out of what was stored
    bench = ZBPPBenchmark(torch.device("cpu"), torch.float32)
    assert bench.validate_gradient_decomposition(8, 16, 12) is True
    assert bench.validate_schedule_optimality(4, 8) is True and bench.validate_memory_compliance(4, 8, 256) is True
    stages = [PipelineStageModule(nn.Sequential(nn.Linear(8, 8), nn.Tanh()), i, decomposer, memory, torch.float32)
              for i in range(2)]
    config = ScheduleConfig(2, 4, 1 << 30, [StageProfile(100., 100., 100., 1, 0, 0., 0.) for _ in range(2)])
    optimizer = ZBPPOptimizer([p for s in stages for p in s.parameters()], lr=1e-2, use_triton=True)
    engine = ZBPPRuntimeEngine(stages, config, optimizer, rank=0, world_size=1, device=torch.device("cpu"),
                               dtype=torch.float32)
    batches = [torch.randn(3, 8) for _ in range(4)]
    labels = [torch.randn(3, 8) for _ in range(4)]
    first = engine.train_step(batches, labels, nn.functional.mse_loss)
    second = engine.train_step(micro_batches=batches, labels=labels)
    assert set(first) >= {"loss", "bubble_fraction", "throughput_samples_per_s"} and second["loss"] < first["loss"]
    with pytest.raises(ValueError):
        engine.train_step(micro_batches=batches[:2], labels=labels[:2])
    assert engine.profile_stage(batches[0], 1, 2).forward_us > 0
    pipe = ZeroBubblePipeline(nn.Sequential(*[nn.Linear(8, 8) for _ in range(4)]), 2, 4)
    assert torch.is_tensor(pipe.train_step(torch.randn(8, 8), torch.randn(8, 8)))
    assert "loss" in pipe.train_step(micro_batches=batches, labels=labels, loss_fn=nn.functional.l1_loss)
    assert pipe.engine.loss_fn is nn.functional.l1_loss
    pipe.train_step(torch.randn(8, 8), torch.randn(8, 8))
    assert pipe.engine.loss_fn is not nn.functional.l1_loss                    # the per-step loss did not stick
    assert len(pipe.profile_stages(batches[0], num_warmup=1, num_iterations=1)) == 2
    assert ModelPartitioner(nn.Sequential(*[nn.Linear(8, 8) for _ in range(4)]), 2, balance_metric="layers").costs == [1.0] * 4
    assert stages[0](input_tensor=batches[0], microbatch_id=7).shape == (3, 8)
    assert memory.retrieve_activation(7, "stage_0_input").shape == (3, 8)


def test_kernel_modules_take_the_reference_forms():
    from trainscale_b200.kernels import (FP8Config, FP8Linear, FP8ScaleManager, FlashAttention, FlashAttentionConfig,
                                         FlexAttention, FlexAttentionConfig, MultiHeadFlashAttention, RMSNorm,
                                         TritonGeGLU, TritonSwiGLU)
    torch.manual_seed(0)
    x = torch.randn(2, 3, 16)
    plain = RMSNorm(16, 1e-6, False)
    assert plain.weight is None and not list(plain.parameters())
    assert torch.allclose(plain(X=x), RMSNorm(16, elementwise_affine=True)(x), atol=1e-6)
    geglu = TritonGeGLU(16, 32, True, False)
    assert geglu.activation == "gelu" and geglu.b_down.shape == (16,) and geglu(x).shape == x.shape
    assert TritonSwiGLU(16, 32, bias=True)(x).shape == x.shape
    attn = FlashAttention(head_dim=8, num_heads=4, num_kv_heads=2, causal=True, dropout=0.0, sliding_window=None)
    q, k, v = torch.randn(2, 4, 6, 8), torch.randn(2, 2, 6, 8), torch.randn(2, 2, 6, 8)
    want = torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1),
                                                            is_causal=True)
    assert torch.allclose(attn(q, k, v), want, atol=1e-5)                       # heads-first layout in and out
    assert torch.allclose(attn(query=q, key=k, value=v), want, atol=1e-5)
    native = FlashAttention(FlashAttentionConfig())
    assert torch.allclose(native(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2), want, atol=1e-5)
    flex = FlexAttention(FlexAttentionConfig(num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                                             query_pre_attn_scalar=8))
    merged = flex(Q=q, K=k, V=v, attention_mask=None, is_causal=True, use_inference_mode=False)
    assert torch.allclose(merged, want.transpose(1, 2).reshape(2, 6, 32), atol=1e-5)
    layer = MultiHeadFlashAttention(embed_dim=32, num_heads=4, num_kv_heads=2, dropout=0.0, bias=True, causal=True,
                                    sliding_window=None)
    tokens = torch.randn(2, 6, 32)
    full = layer(tokens)
    wq, wk, wv = layer.wqkv.split((32, 16, 16))
    bq, bk, bv = layer.bqkv.split((32, 16, 16))
    key_cache = (tokens[:, :5] @ wk.t() + bk).view(2, 5, 2, 8).transpose(1, 2)
    value_cache = (tokens[:, :5] @ wv.t() + bv).view(2, 5, 2, 8).transpose(1, 2)
    last = layer(query=tokens[:, 5:], key=tokens[:, 5:], value=tokens[:, 5:], key_cache=key_cache, value_cache=value_cache)
    assert torch.allclose(last, full[:, 5:], atol=1e-5)                         # decoding behind a cache == full pass
    assert torch.allclose(layer(tokens, tokens, tokens), full, atol=1e-5)
    assert MultiHeadFlashAttention(32, 4).bqkv is None
    assert FP8Linear(128, 16, False, 128)(X=torch.randn(2, 128, dtype=torch.bfloat16)).shape == (2, 16)
    with pytest.raises(ValueError):
        FP8Linear(128, 16, block_size=64)
    assert FP8ScaleManager(FP8Config(), "cpu").device == "cpu"


def test_remaining_reference_forms_of_shared_classes():
    import torch.nn as nn
    import torch._inductor.config as inductor
    from trainscale_b200.benchmark_suite import BenchmarkSuite
    from trainscale_b200.kernels.compat import InductorConfig
    from trainscale_b200.losses import ChunkedCrossEntropyLoss, HuberLoss
    from trainscale_b200.metrics.throughput import ThroughputTracker
    from trainscale_b200.parallel.activation import ActivationCheckpointConfig, HierarchicalCheckpointManager
    from trainscale_b200.parallel.dist_kernels import DistributedKernels, GradientCompressor, ZeroCopyTransfer
    from trainscale_b200.parallel.grad_buffer import ParamAndGradBucketGroup, ParamAndGradBuffer
    from trainscale_b200.parallel.mesh import MeshCache, ParallelDims, ParallelDimsConfig
    from trainscale_b200.registry import DependencyGraph, KernelPatcher
    from trainscale_b200.utils.cuda_graphs import InductorConfigManager, ModelCompiler
    from types import SimpleNamespace

    graph = DependencyGraph()
    graph.add_module(name="a", dependencies=["b"])
    assert graph.edges == {"a": {"b"}, "b": set()}
    lin = nn.Linear(2, 2)
    assert KernelPatcher().patch(lin, model_info=None) is lin
    tracker = ThroughputTracker()
    assert tracker.compute_mfu(flops_per_token=1e9, seq_len=128) == 0.0           # nothing measured yet
    tracker.load_state_dict(state=tracker.state_dict())
    z, y = torch.randn(10, 7), torch.randint(0, 7, (10,))
    assert torch.allclose(ChunkedCrossEntropyLoss(chunk_size=4)(logits=z, labels=y), nn.functional.cross_entropy(z, y))
    assert float(HuberLoss()(pred=z, target=z + 1)) == 0.5
    before = inductor.max_autotune
    InductorConfigManager.apply(InductorConfig(max_autotune=not before))          # the class-level form of the reference
    assert inductor.max_autotune != before
    InductorConfigManager.restore()
    assert inductor.max_autotune == before
    assert InductorConfigManager(max_autotune=True).apply() == {}                 # recorded only unless asked to apply
    assert ModelCompiler().compile(lin, example_inputs=torch.randn(1, 2))(torch.ones(1, 2)).shape == (1, 2)
    copies = ZeroCopyTransfer(16)
    assert copies.staging_bytes == 16 * 2 ** 20 and copies.host_to_device(x=z, device=None, use_pool=False) is z
    assert BenchmarkSuite().run_rms_norm([4], [2048], [4096]) == [] or torch.cuda.is_available()
    planner = HierarchicalCheckpointManager(config=ActivationCheckpointConfig(), num_layers=12)
    assert planner.num_layers == 12 and not planner.layers

    dims = ParallelDims(config=ParallelDimsConfig(world_size=1))
    assert dims.config.world_size == 1
    MeshCache.set("tp", "mesh-of-tp")
    assert MeshCache.get("tp") == "mesh-of-tp" and MeshCache.get(name="absent") is None
    ddp = SimpleNamespace(use_distributed_optimizer=False, overlap_grad_reduce=False, average_in_collective=True)
    names = {p: n for n, p in lin.named_parameters()}
    buffer = ParamAndGradBuffer(ddp, torch.float32, torch.float32, list(lin.parameters()), None, 1000, names, 0.5)
    assert buffer.numel_unpadded == 6 and buffer.gradient_scaling_factor == 0.5 and len(buffer.param_to_name) == 2
    group = ParamAndGradBucketGroup(buffer.buckets, ddp, None, 1)
    assert group.overlap_grad_reduce is False and group.average is True
    with pytest.raises(ValueError):
        ParamAndGradBucketGroup(buffer.buckets, ddp_config=ddp, collective_group=None, collective_group_size=2)

    kernels = DistributedKernels()                                                # no process group: identities
    t = torch.ones(4, 2)
    assert kernels.sequence_parallel_all_gather(x=t, dim=1, group=None, async_op=False) is t
    out = torch.empty(4, 2)
    assert float(kernels.reduce_scatter(output=out, input_tensors=[t * 2]).sum()) == 16.0
    assert kernels.all_gather_into_tensor(None, input_tensor=t) is t and kernels.broadcast_object_list(object_list=[1]) == [1]
    compressor = GradientCompressor(use_fp16=True)
    payload, meta = compressor.compress(t, tensor_id=3)
    assert compressor.decompress(tensor=payload[0], metadata=meta).dtype is torch.float32


def test_optimizer_scheduler_and_callback_options_of_the_reference():
    from trainscale_b200 import callbacks as C
    from trainscale_b200 import optim as O
    from trainscale_b200 import schedulers as S
    lin = nn.Linear(4, 4)
    opt = O.AdamW(lin.parameters(), lr=1e-2, use_triton=False, max_grad_norm=1.0, grad_accumulation_steps=1)
    lin(torch.randn(2, 4)).sum().backward()
    opt.step()
    O.AdamW(lin.parameters(), use_triton=True)                                  # implementation switch: same maths, no effect
    O.LAMB(lin.parameters(), trust_ratio_clip=5.0)
    O.SophiaG(lin.parameters(), hessian_update_interval=5)
    sched = S.BaseScheduler(opt, 100, warmup_ratio=0.1, warmup_start_lr=0.0, min_lr=1e-4, last_epoch=-1)
    assert sched.warmup_steps == 10
    rex = S.REXScheduler(opt, 100, gamma=0.9)
    rex.step(step=50)
    S.InverseSquareRootScheduler(opt, 100, warmup_steps=10, warmup_init_lr=1e-7)
    stop = C.EarlyStoppingCallback(patience=1, monitor="eval_loss", min_delta=0.1, mode="min", restore_best=False)
    assert stop.metric == "eval_loss" and stop.threshold == 0.1
    handler = C.CallbackHandler()
    seen = []

    class Probe(C.Callback):
        def on_step_end(self, ctx):
            seen.append("step")

    probe = Probe()
    handler.add_callback(probe)
    handler.trigger("on_step_end", C.CallbackContext())
    handler.remove_callback(probe)
    handler.trigger("on_step_end", C.CallbackContext())
    assert seen == ["step"]
    assert C.ProgressCallback(refresh_rate=5).refresh_rate == 5


def test_checkpoint_manager_and_trainer_take_the_reference_forms(tmp_path):
    from trainscale_b200.hub import CheckpointManager
    from trainscale_b200.trainer.base import Trainer
    from trainscale_b200.config.training_args import TrainingArguments
    lin = nn.Linear(4, 2)
    manager = CheckpointManager(save_dir=str(tmp_path / "ckpts"), hub_manager=None, max_checkpoints=2)
    results = [manager.save(lin, step=s, loss=1.0 / (s + 1)) for s in (1, 2, 3)]
    assert all(r.is_ok() for r in results)
    latest = manager.get_latest_checkpoint()
    assert latest is not None and "3" in str(latest)
    assert len([p for p in (tmp_path / "ckpts").iterdir() if p.is_dir()]) <= 2    # the bound is kept

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(4, 2)

        def forward(self, x):
            return self.lin(x)

    net = Net()
    data = [{"x": torch.randn(4), "labels": torch.randn(2)} for _ in range(8)]

    def collate(rows):
        return {k: torch.stack([r[k] for r in rows]) for k in ("x", "labels")}

    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    args = TrainingArguments(output_dir=str(tmp_path / "run"), per_device_train_batch_size=4, num_train_epochs=1,
                             max_steps=2, logging_steps=1, save_strategy="no")
    trainer = Trainer(net, args, train_dataset=data, eval_dataset=data, data_collator=collate, optimizers=(opt, None),
                      loss_fn=nn.functional.mse_loss)
    assert next(iter(trainer.get_train_dataloader()))["x"].shape == (4, 4)
    before = net.lin.weight.detach().clone()
    trainer.train()
    assert not torch.equal(before, net.lin.weight.detach())


def test_tensor_parallel_layers_build_without_a_context_and_managers_take_configs():
    from trainscale_b200.parallel.dist_utils import DistributedManager, GradientSynchronizer
    from trainscale_b200.parallel.tp import (ColumnParallelLinear, ParallelMLP, ProcessGroupManager, RowParallelLinear,
                                             TensorParallelConfig, VocabParallelEmbedding)
    col = ColumnParallelLinear(16, 8, bias=True, init_method=lambda w: nn.init.constant_(w, 0.5))
    assert float(col.weight.detach().mean()) == 0.5                             # one rank: the whole layer, initialised as asked
    x = torch.randn(2, 16)
    row = RowParallelLinear(8, 16, init_method=nn.init.zeros_)
    assert row(col(x)).abs().sum() == 0
    with pytest.raises(NotImplementedError):
        ColumnParallelLinear(16, 8, skip_bias_add=True)
    emb = VocabParallelEmbedding(32, 8, padding_idx=0)
    assert emb(torch.tensor([[0, 3]]))[0, 0].abs().sum() == 0                   # the padding row is zero
    mlp = ParallelMLP(16, 32, use_gated=True, dropout_prob=0.0)
    assert mlp(hidden_states=x).shape == x.shape
    groups = ProcessGroupManager.get()
    groups.initialize(TensorParallelConfig())
    buf = groups.acquire_buffer(torch.float32, 16)
    assert buf.shape == (16,)
    groups.release_buffer(buffer=buf)
    manager = DistributedManager(config=None)
    assert manager.world_size == 1
    sync = GradientSynchronizer(model=nn.Linear(2, 2), bucket_size_mb=1.0, async_sync=False)
    sync.sync_gradients()


def test_factory_functions_take_the_reference_positional_order():
    """Factories whose leading arguments come in another order in the reference recognise that order by type."""
    import torch.nn as nn
    from trainscale_b200.config.sota_config import LossConfig, OptimizerConfig
    from trainscale_b200.data.collate import create_causal_lm_collate
    from trainscale_b200.data.length_manager import create_content_distributor
    from trainscale_b200.kernels import create_causal_mask, create_sliding_window_causal_mask
    from trainscale_b200.losses import create_loss
    from trainscale_b200.optim import create_optimizer
    from trainscale_b200.parallel.dist_utils import DistributedState, prepare_model_for_distributed
    from trainscale_b200.schedulers import create_scheduler
    lin = nn.Linear(4, 4)
    opt = create_optimizer("adamw", lin.parameters(), 1e-3, 0.1)                 # (name, params, lr, weight_decay)
    assert type(opt).__name__ == "AdamW" and opt.param_groups[0]["lr"] == 1e-3 and opt.param_groups[0]["weight_decay"] == 0.1
    assert type(create_optimizer(lin.parameters(), OptimizerConfig())).__name__ == "AdamW"
    sgd = torch.optim.SGD(lin.parameters(), lr=0.1)
    assert type(create_scheduler("cosine", sgd, 100, 10)).__name__ == "CosineScheduler"      # (name, optimizer, ...)
    assert type(create_scheduler(sgd, "linear", 100)).__name__ == "LinearScheduler"
    assert isinstance(create_loss(LossConfig()), nn.Module) and type(create_loss("focal")).__name__ == "FocalLoss"
    assert create_content_distributor(128, "proportional").available_tokens <= 128          # (max_length, mode)
    assert type(create_causal_lm_collate(0, 128, "right")).__name__ == "CollateFn"          # (pad, max_length, side)
    assert type(create_causal_lm_collate(0, True)).__name__ == "_ShiftedCollate"
    model, engine = prepare_model_for_distributed(lin, DistributedState(), "single")         # (model, state, strategy)
    assert model is lin and engine is None
    assert create_causal_mask(4, torch.float32, "cpu").shape == (4, 4)                       # (n, dtype, device)
    assert create_sliding_window_causal_mask(4, 2, torch.float32, "cpu")[3, 0] == float("-inf")


def test_region_functions_and_seed_take_the_reference_positional_order():
    from trainscale_b200.parallel.dist_utils import DistributedState, set_deterministic_seed
    from trainscale_b200.parallel.tp import (all_gather_from_sequence_parallel_region, copy_to_tensor_parallel_region,
                                             gather_from_tensor_parallel_region)
    x = torch.randn(4, 8)
    assert set_deterministic_seed(1, DistributedState(), True, False) == 1 and set_deterministic_seed(1, 3) == 4
    assert copy_to_tensor_parallel_region(x, False) is x                     # (input_, async_op) on one rank: identity
    assert gather_from_tensor_parallel_region(x, -1) is x and gather_from_tensor_parallel_region(x, 1) is x
    assert all_gather_from_sequence_parallel_region(x, 0) is x
    with pytest.raises(NotImplementedError):
        gather_from_tensor_parallel_region(x, 0)                             # another dimension is not silently ignored


def test_estimators_take_the_reference_positional_order():
    import torch.nn as nn
    from trainscale_b200.parallel.cp import estimate_memory_per_gpu
    from trainscale_b200.parallel.pipeline import balance_stages_by_memory
    from trainscale_b200.quantization import estimate_memory_usage
    assert estimate_memory_usage(7.0, None)["model_gb"] == pytest.approx(7e9 * 2 / 2 ** 30, abs=0.01)   # no config: 16 bit
    chain = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 8))
    assert balance_stages_by_memory(chain, 2, (2, 8)) == [range(0, 1), range(1, 2)]                  # (model, n, input_shape)
    by_position = estimate_memory_per_gpu(1, 8192, 4096, 32, 2)                                       # (b, s, h, heads, cp)
    assert isinstance(by_position, int)
    assert by_position == estimate_memory_per_gpu(batch_size=1, seq_len=8192, hidden_dim=4096, num_heads=32, cp_degree=2)
    assert estimate_memory_per_gpu(8192, 2, 4096, 1, 8, 128)["tokens_per_gpu"] == 4096                # the native form


def test_pack_sequences_takes_the_reference_positional_columns():
    from trainscale_b200.data.packing import pack_sequences
    ids = torch.tensor([[5, 6, 0, 0], [7, 0, 0, 0]])
    mask = (ids != 0).long()
    by_position = pack_sequences(ids, mask, ids.clone(), 8, 0)               # (input_ids, attention_mask, labels, max, pad)
    by_name = pack_sequences(input_ids=ids, attention_mask=mask, labels=ids.clone(), max_length=8, pad_token_id=0)
    assert by_position[0]["input_ids"].tolist() == [5, 6, 7, 0, 0, 0, 0, 0]
    assert all(torch.equal(by_position[0][k], by_name[0][k]) for k in by_name[0] if torch.is_tensor(by_name[0][k]))
    assert pack_sequences([{"input_ids": torch.tensor([1, 2])}], 4)[0]["input_ids"].tolist() == [1, 2, 0, 0]   # native form
    assert pack_sequences([torch.tensor([1, 2]), torch.tensor([3])], None, None, 4)[0]["input_ids"].tolist() == [1, 2, 3, 0]
