import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_decode_attention_matches_reference():
    import ctypes
    from trainscale_b200.ops import _lib
    from trainscale_b200.ops.attention import attention_reference
    torch.manual_seed(0)
    dev = "cuda"
    lib = _lib.load("decode")
    n, Hq, Hkv, D, bs = 3, 8, 2, 128, 16
    lens = [5, 700, 1300]
    nb = sum(-(-l // bs) for l in lens) + 4
    kc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    perm = torch.randperm(nb).tolist()
    maxb = max(-(-l // bs) for l in lens)
    bt = torch.zeros(n, maxb, dtype=torch.int32)
    used = 0
    for i, l in enumerate(lens):
        k = -(-l // bs)
        bt[i, :k] = torch.tensor(perm[used:used + k], dtype=torch.int32)
        used += k
    bt = bt.to(dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    q = torch.randn(n, Hq * D, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    chunk = 512
    splits = -(-max(lens) // chunk)
    po = torch.empty(n, Hq, splits, D, device=dev)
    pl = torch.empty(n, Hq, splits, device=dev)
    rc = lib.ts_decode_attention(_lib.ptr(q), Hq * D, _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(bt), maxb, _lib.ptr(sl),
                                 _lib.ptr(out), Hq * D, _lib.ptr(po), _lib.ptr(pl), n, Hq, Hkv, D, bs, chunk, splits,
                                 ctypes.c_float(1 / math.sqrt(D)), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    for i, l in enumerate(lens):
        idx = bt[i, :-(-l // bs)].long()
        k = kc[idx].reshape(-1, Hkv, D)[:l].unsqueeze(0)
        v = vc[idx].reshape(-1, Hkv, D)[:l].unsqueeze(0)
        ref = attention_reference(q[i].view(1, 1, Hq, D), k, v, True).reshape(-1)
        assert (out[i].float() - ref.float()).abs().max().item() < 2e-2


def test_engine_on_gpu_matches_full_forward_logits():
    from trainscale_b200.inference import CacheConfig, EngineConfig, GenerationParams, SOTAInferenceEngine
    from trainscale_b200.models.llama import LlamaConfig, build_model
    cfg = LlamaConfig(vocab_size=300, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=1)
    eng = SOTAInferenceEngine(EngineConfig(model="tiny", cache=CacheConfig(block_size=16, num_gpu_blocks=256,
                                                                            max_model_len=512)), model=model)
    prompts = ["the quick brown fox jumps over the lazy dog " * 3, "hello"]
    res = eng.generate(prompts, GenerationParams(max_tokens=16, temperature=0.0, ignore_eos=True)).unwrap()
    tok = eng.core.tokenizer
    for p, r in zip(prompts, res):
        assert len(r.token_ids) == 16
        # teacher-forced check: the full-context forward ranks each generated token (near) first
        ids = [tok.bos_token_id] + tok.encode_raw(p) + r.token_ids
        with torch.no_grad():
            logits = model(torch.tensor([ids], device="cuda")).logits[0].float()
        n0 = len(ids) - 16
        for j, t in enumerate(r.token_ids):
            row = logits[n0 - 1 + j]
            assert row[t] >= row.max() - 0.15, (j, row[t].item(), row.max().item())


def test_cuda_graph_decode_matches_eager_decode():
    """The decode loop replayed from CUDA graphs (padded batch, spare cache block for the padding rows) produces the
    tokens of the eager loop, for a batch whose size is not a power of two and that shrinks as requests finish."""
    from trainscale_b200.inference import CacheConfig, EngineConfig, GenerationParams, SOTAInferenceEngine
    from trainscale_b200.models.llama import LlamaConfig, build_model
    from trainscale_b200.ops import _lib
    cfg = LlamaConfig(vocab_size=300, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64)
    prompts = [[5, 9, 200, 31, 77, 12] * 5, [8, 8, 101], [250, 3, 3, 3, 19, 44, 60, 2, 91] * 12, [17] * 40, [4, 5]]
    lens = [24, 9, 30, 17, 12]

    def run(eager):
        model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=1)
        eng = SOTAInferenceEngine(EngineConfig(model="tiny", enforce_eager=eager,
                                               cache=CacheConfig(block_size=16, num_gpu_blocks=256, max_model_len=512)),
                                  model=model)
        reqs = [eng.core.add_request(p, GenerationParams(max_tokens=n, temperature=0.0, ignore_eos=True))
                for p, n in zip(prompts, lens)]
        while eng.core.has_unfinished():
            eng.core.step()
        return [r.output_ids for r in reqs], eng

    want, _ = run(True)
    got, eng = run(False)
    assert eng.core.runner.graph_replays > 20 and len(eng.core.runner.graphs) >= 2
    torch.cuda.synchronize()
    _lib.raise_on_any_device_error()
    agree = sum(g == w for g, w in zip(got, want))
    # identical kernels on identical inputs: the sequences must be the same (a near-tie may flip at most one of them)
    assert agree >= len(want) - 1, (got, want)
    for g, w in zip(got, want):
        assert g[:6] == w[:6]
