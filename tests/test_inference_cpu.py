"""Inference engine on CPU: greedy decoding through the paged cache equals a plain full-context forward,
continuous batching with chunked prefill is order-independent, prefix caching reuses blocks, streaming works."""
import asyncio

import torch

from trainscale_b200.inference import (CacheConfig, EngineConfig, GenerationParams, SchedulerConfig,
                                       SOTAAsyncStreamEngine, SOTAInferenceEngine, create_openai_server)
from trainscale_b200.models.llama import LlamaConfig, build_model

CFG = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=16)


def make(seqs=8, budget=64, block=4):
    model = build_model(CFG, dtype=torch.float32, seed=1)
    cfg = EngineConfig(model="tiny", device="cpu", dtype="float32",
                       scheduler=SchedulerConfig(max_num_seqs=seqs, max_num_batched_tokens=budget),
                       cache=CacheConfig(block_size=block, num_gpu_blocks=256, max_model_len=256))
    return SOTAInferenceEngine(cfg, model=model), model


def greedy_reference(model, ids, n):
    ids = list(ids)
    for _ in range(n):
        with torch.no_grad():
            logits = model(torch.tensor([ids])).logits[0, -1]
        ids.append(int(logits.argmax()))
    return ids


def test_greedy_matches_full_forward():
    eng, model = make()
    prompt = "hello world"
    r = eng.generate(prompt, GenerationParams(max_tokens=8, temperature=0.0, ignore_eos=True)).unwrap()
    ids = [eng.core.tokenizer.bos_token_id] + eng.core.tokenizer.encode_raw(prompt)
    assert r.token_ids == greedy_reference(model, ids, 8)[len(ids):]
    assert r.metrics.ttft is not None and r.metrics.completion_tokens == 8 and r.finish_reason == "length"


def test_batching_and_chunked_prefill_are_order_independent():
    prompts = ["a" * 50, "bc", "the quick brown fox", "x" * 23]
    p = GenerationParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    eng1, _ = make(seqs=8, budget=16)      # tiny token budget -> prompts are prefilled in chunks
    out1 = [r.token_ids for r in eng1.generate(prompts, p).unwrap()]
    eng2, _ = make(seqs=1, budget=512)     # one request at a time
    out2 = [r.token_ids for r in eng2.generate(prompts, p).unwrap()]
    assert out1 == out2
    assert eng1.core.steps > eng2.core.steps / 4


def test_prefix_cache_reuses_blocks_and_keeps_outputs():
    eng, _ = make(block=4)
    p = GenerationParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    a = eng.generate("shared prefix 0123456789 tail A", p).unwrap()
    before = eng.core.cache.prefix_hits
    b = eng.generate("shared prefix 0123456789 tail A", p).unwrap()
    assert eng.core.cache.prefix_hits > before
    assert a.token_ids == b.token_ids
    assert eng.core.cache.alloc.num_free == 256


def test_sampling_is_seeded_and_stops():
    eng, _ = make()
    p = GenerationParams(max_tokens=12, temperature=1.0, top_k=20, top_p=0.9, seed=7, ignore_eos=True)
    a = eng.generate("seed me", p).unwrap().token_ids
    b = eng.generate("seed me", p).unwrap().token_ids
    assert a == b
    stop_id = a[3]
    c = eng.generate("seed me", GenerationParams(max_tokens=12, temperature=1.0, top_k=20, top_p=0.9, seed=7,
                                                 stop_token_ids=[stop_id])).unwrap()
    assert c.finish_reason == "stop" and len(c.token_ids) <= 4


def test_async_stream_and_server_app():
    model = build_model(CFG, dtype=torch.float32, seed=1)
    cfg = EngineConfig(model="tiny", device="cpu", dtype="float32", cache=CacheConfig(block_size=4, num_gpu_blocks=128,
                                                                                      max_model_len=128))
    eng = SOTAAsyncStreamEngine(cfg, model=model)

    async def go():
        chunks = []
        async for ch in eng.generate_stream("stream", GenerationParams(max_tokens=5, temperature=0.0, ignore_eos=True)):
            chunks.append(ch)
        return chunks

    chunks = asyncio.run(go())
    assert len(chunks) == 5 and chunks[-1].finished and chunks[-1].finish_reason == "length"
    app = create_openai_server(eng)
    paths = {r.path for r in app.routes}
    assert {"/v1/completions", "/v1/chat/completions", "/health", "/metrics"} <= paths


def _tiny_lm(seed, layers=2, vocab=97):
    from trainscale_b200.models.llama import LlamaConfig, build_model
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=64, intermediate_size=128, num_hidden_layers=layers,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=256)
    return build_model(cfg, dtype=torch.float32, device="cpu", seed=seed).eval()


def test_speculative_greedy_equals_target_greedy():
    from trainscale_b200.inference.speculative import greedy_generate, speculative_generate
    target, draft = _tiny_lm(1), _tiny_lm(2, layers=1)
    prompt = [5, 17, 3, 42, 8]
    want = greedy_generate(target, prompt, 24)
    got, stats = speculative_generate(target, draft, prompt, 24, k=4)
    assert got == want
    assert stats.proposed > 0 and 0.0 <= stats.acceptance_rate <= 1.0
    # a draft identical to the target is always accepted: k + 1 tokens per target forward
    got2, stats2 = speculative_generate(target, target, prompt, 24, k=3)
    assert got2 == want and stats2.acceptance_rate == 1.0
    assert stats2.target_forwards <= 1 + (24 + 3) // 4 + 1


def test_speculative_sampling_runs_and_respects_eos():
    from trainscale_b200.inference.speculative import speculative_generate
    target, draft = _tiny_lm(1), _tiny_lm(3, layers=1)
    g = torch.Generator().manual_seed(0)
    out, stats = speculative_generate(target, draft, [1, 2, 3], 16, k=3, temperature=0.8, generator=g)
    assert 1 <= len(out) <= 16 and all(0 <= t < 97 for t in out)
    out2, _ = speculative_generate(target, draft, [1, 2, 3], 16, k=3, temperature=0.0, eos_token_id=out[0])
    assert len(out2) >= 1


def test_lora_adapter_registry_switches_weights():
    from trainscale_b200.inference.speculative import LoRAAdapterRegistry
    from trainscale_b200.lora import get_peft_model
    m = get_peft_model(_tiny_lm(4), r=4, lora_alpha=8.0)
    ids = torch.tensor([[3, 9, 27, 81]])
    reg = LoRAAdapterRegistry(m, max_loras=2)
    base = m(input_ids=ids).logits.clone()
    for name, seed in (("a", 10), ("b", 11), ("c", 12)):
        torch.manual_seed(seed)
        for n, p in m.named_parameters():
            if n.endswith("lora_B"):
                p.data.normal_(std=0.05)
        reg.register(name)
    outs = {}
    for name in ("a", "b", "c", "a"):
        reg.activate(name)
        outs.setdefault(name, []).append(m(input_ids=ids).logits.clone())
    assert not torch.allclose(outs["a"][0], outs["b"][0]) and not torch.allclose(outs["b"][0], outs["c"][0])
    assert torch.allclose(outs["a"][0], outs["a"][1])         # came back from the offloaded copy unchanged
    reg.activate(None)
    assert torch.allclose(m(input_ids=ids).logits, base, atol=1e-6)
    groups = reg.group_requests(["a", None, "b", "a", None])
    assert groups[0][0] is None and sorted(i for _, g in groups for i in g) == [0, 1, 2, 3, 4]


def test_engine_generate_with_speculative_config_matches_plain_engine():
    from trainscale_b200.inference.engine import EngineConfig, GenerationParams, SOTAInferenceEngine
    target, draft = _tiny_lm(1, vocab=300), _tiny_lm(2, layers=1, vocab=300)   # the byte tokenizer's id range
    cfg = EngineConfig()
    plain = SOTAInferenceEngine(cfg, model=target)
    params = GenerationParams(max_tokens=12, temperature=0.0)
    want = plain.generate("hello world", params).unwrap()
    cfg2 = EngineConfig()
    cfg2.speculative.enabled = True
    cfg2.speculative.num_speculative_tokens = 3
    spec = SOTAInferenceEngine(cfg2, model=target, draft_model=draft)
    got = spec.generate("hello world", params).unwrap()
    assert got.token_ids == want.token_ids
    assert 0.0 <= got.speculative_acceptance <= 1.0


def test_mixed_adapter_batch_matches_merged_models():
    """Requests with adapter a, adapter b and no adapter share one continuous batch; each gets exactly the tokens that a
    model with its adapter merged into the weights produces.  Two of the prompts are equal: the prefix cache must not
    hand K/V computed under one adapter to a request that uses another."""
    import copy
    import torch
    from trainscale_b200.inference.engine import EngineConfig, EngineCore, GenerationParams, LoRAServingConfig
    from trainscale_b200.lora import get_peft_model, lora_state_dict, merge_and_unload
    from trainscale_b200.models.llama import LlamaConfig, build_model
    cfg = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16)
    base = build_model(cfg, dtype=torch.float32, device="cpu", seed=0)
    m = copy.deepcopy(base)
    get_peft_model(m, r=4)
    adapters = {}
    for name, seed in (("a", 1), ("b", 2)):
        g = torch.Generator().manual_seed(seed)
        for n, p in m.named_parameters():
            if "lora_" in n:
                p.data = torch.randn(p.shape, generator=g) * 0.2
        adapters[name] = lora_state_dict(m)
    ec = EngineConfig(model="custom", tokenizer="byte", device="cpu", dtype="float32", lora=LoRAServingConfig(max_loras=4))

    def run(model, reqs, ad=None):
        eng = EngineCore(ec, model=model)
        if ad:
            eng.load_adapters(ad)
        rs = [eng.add_request(p, GenerationParams(max_tokens=6, temperature=0.0, lora_name=a)) for p, a in reqs]
        while eng.has_unfinished():
            eng.step()
        return [r.output_ids for r in rs]

    prompts = [list(range(5, 45)), list(range(40, 52)), list(range(5, 45))]
    mixed = run(m, list(zip(prompts, ("a", "b", None))), adapters)
    for p, a, got in zip(prompts, ("a", "b", None), mixed):
        mm = copy.deepcopy(base)
        if a:
            get_peft_model(mm, r=4)
            for n, q in mm.named_parameters():
                if n in adapters[a]:
                    q.data = adapters[a][n].clone()
            merge_and_unload(mm)
        assert run(mm, [(p, None)])[0] == got
    assert mixed[0] != mixed[2]
    import pytest
    with pytest.raises(ValueError):
        EngineCore(EngineConfig(model="custom", tokenizer="byte", device="cpu", dtype="float32"), model=m).load_adapters(adapters)


def test_tensor_parallel_serving_matches_single_process():
    import subprocess
    import sys
    from pathlib import Path
    case = Path(__file__).parent / "dist_cases" / "inference_tp.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29695", str(case)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT inference tp=2" in r.stdout and "ok=True" in r.stdout
