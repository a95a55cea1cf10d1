"""Losses, schedulers, optimizers, callbacks, hub/checkpoint manager, registry, metrics, LoRA, quantisation, RL utils."""
import math

import pytest
import torch
import torch.nn.functional as F

from trainscale_b200 import losses as L
from trainscale_b200.callbacks import CallbackContext, CallbackHandler, Callback, CheckpointCallback, EarlyStoppingCallback
from trainscale_b200.hub import CheckpointManager, CircuitBreaker, ModelDeserializer, ModelSerializer, RetryPolicy, execute_with_retry
from trainscale_b200.core.errors import CheckpointLoadError, HubError
from trainscale_b200.schedulers import create_scheduler


def test_dpo_family_formulas():
    pc, pr, rc, rr = torch.tensor([-5.0, -3.0]), torch.tensor([-6.0, -2.5]), torch.tensor([-5.5, -3.0]), torch.tensor([-5.8, -2.9])
    x = (pc - pr) - (rc - rr)
    loss, cr, rjr = L.DPOLoss(0.1)(pc, pr, rc, rr)
    assert torch.allclose(loss, -F.logsigmoid(0.1 * x).mean()) and torch.allclose(cr, 0.1 * (pc - rc))
    assert torch.allclose(L.DPOLoss(0.1, "hinge")(pc, pr, rc, rr)[0], torch.relu(1 - 0.1 * x).mean())
    assert torch.allclose(L.DPOLoss(0.1, "ipo")(pc, pr, rc, rr)[0], ((x - 5.0) ** 2).mean())
    sm = L.DPOLoss(0.1, label_smoothing=0.2)(pc, pr, rc, rr)[0]
    assert torch.allclose(sm, (-0.8 * F.logsigmoid(0.1 * x) - 0.2 * F.logsigmoid(-0.1 * x)).mean())
    s, _, _ = L.SimPOLoss(2.0, 0.5)(pc, pr, torch.tensor([5.0, 3.0]), torch.tensor([6.0, 2.0]))
    assert torch.allclose(s, -F.logsigmoid(2.0 * (pc / torch.tensor([5.0, 3.0]) - pr / torch.tensor([6.0, 2.0])) - 0.5).mean())
    lp = torch.tensor([-0.5, -0.2])
    assert torch.allclose(L.ORPOLoss.log_odds(lp), lp - torch.log1p(-lp.exp()))


def test_lm_losses_match_torch():
    torch.manual_seed(0)
    lg, lb = torch.randn(2, 5, 11), torch.randint(0, 11, (2, 5))
    lb[0, 0] = -100
    ref = F.cross_entropy(lg.view(-1, 11), lb.view(-1), ignore_index=-100)
    assert torch.allclose(L.CrossEntropyLoss()(lg, lb), ref)
    h, w = torch.randn(10, 16), torch.randn(11, 16)
    assert torch.allclose(L.ChunkedCrossEntropyLoss()(h, w, lb.view(-1)), F.cross_entropy(h @ w.t(), lb.view(-1), ignore_index=-100), atol=1e-5)
    t = torch.randn(2, 5, 11)
    d = L.DistillationLoss(2.0, 0.5)(lg, t, lb)
    valid = lb.view(-1) != -100
    kd = F.kl_div(torch.log_softmax(lg.view(-1, 11)[valid] / 2, -1), torch.softmax(t.view(-1, 11)[valid] / 2, -1), reduction="batchmean") * 4
    assert torch.allclose(d, 0.5 * kd + 0.5 * ref, atol=1e-5)
    assert len(L.LossRegistry.available()) >= 30 and isinstance(L.create_loss("focal"), L.FocalLoss)
    lbl = L.LoadBalancingLoss(4, 1, 1.0)(torch.zeros(8, 4), torch.arange(8) % 4)
    assert abs(float(lbl) - 1.0) < 1e-6        # perfectly balanced routing gives E * sum (1/E * 1/E) = 1


def test_schedulers_shapes():
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    s = create_scheduler(opt, "wsd", 100, warmup_steps=10, min_lr_ratio=0.1, stable_ratio=0.5)
    lrs = []
    for _ in range(100):
        lrs.append(opt.param_groups[0]["lr"])
        s.step()
    assert lrs[0] == pytest.approx(0.1) and lrs[9] == pytest.approx(1.0) and lrs[40] == 1.0 and lrs[-1] < 0.2
    assert all(a >= b - 1e-12 for a, b in zip(lrs[55:], lrs[56:]))
    opt2 = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=2.0)
    c = create_scheduler(opt2, "cosine", 50, warmup_ratio=0.1, min_lr_ratio=0.0)
    assert c.warmup_steps == 5
    for _ in range(50):
        c.step()
    assert opt2.param_groups[0]["lr"] == pytest.approx(0.0, abs=1e-6)
    st = c.state_dict()
    c2 = create_scheduler(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=2.0), "cosine", 50, warmup_steps=5)
    c2.load_state_dict(st)
    assert c2.last_step == c.last_step
    for name in ("linear", "polynomial", "inverse_sqrt", "rex", "cosine_restart", "onecycle", "constant"):
        o = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
        sch = create_scheduler(o, name, 20, warmup_steps=2)
        for _ in range(20):
            sch.step()
            assert math.isfinite(o.param_groups[0]["lr"]) and o.param_groups[0]["lr"] >= 0


def test_callbacks_fire_in_order_and_checkpoint_rotation(tmp_path):
    seen = []

    class Rec(Callback):
        def on_step_end(self, ctx):
            seen.append(ctx.state.global_step)

    class S:
        global_step = 0
    h = CallbackHandler([Rec()])
    ctx = CallbackContext(state=S())
    for i in range(3):
        S.global_step = i + 1
        h.fire("on_step_end", ctx)
    assert seen == [1, 2, 3]
    with pytest.raises(ValueError):
        h.fire("on_nothing", ctx)
    es = EarlyStoppingCallback(patience=2)
    for v in (1.0, 0.9, 0.95, 0.96):
        ctx.metrics = {"eval_loss": v}
        es.on_evaluate(ctx)
    assert ctx.should_stop
    for s in (10, 20, 30, 40):
        (tmp_path / f"checkpoint-{s}").mkdir()
    (tmp_path / "checkpoint-best").mkdir()
    CheckpointCallback(str(tmp_path), save_total_limit=2).cleanup_old_checkpoints()
    assert sorted(p.name for p in tmp_path.iterdir()) == ["checkpoint-30", "checkpoint-40", "checkpoint-best"]


def test_serializer_integrity_retry_and_manager(tmp_path):
    sd = {f"w{i}": torch.randn(64, 64) for i in range(6)}
    info = ModelSerializer(max_shard_bytes=40000).save(sd, tmp_path / "m")
    assert len(info["files"]) > 1
    back = ModelDeserializer().load(tmp_path / "m")
    assert all(torch.equal(back[k], sd[k]) for k in sd)
    shard = tmp_path / "m" / info["files"][0]
    data = bytearray(shard.read_bytes())
    data[-1] ^= 0xFF
    shard.write_bytes(bytes(data))
    with pytest.raises(CheckpointLoadError):
        ModelDeserializer().load(tmp_path / "m")
    calls = {"n": 0}

    def flaky():
        calls["n"] += 1
        if calls["n"] < 3:
            raise OSError("transient")
        return "ok"
    assert execute_with_retry(flaky, RetryPolicy(max_attempts=4, base_delay=0), sleep=lambda s: None) == "ok"
    br = CircuitBreaker(failure_threshold=2, reset_timeout=10, clock=lambda: 0.0)
    with pytest.raises(HubError):
        execute_with_retry(lambda: (_ for _ in ()).throw(OSError("down")), RetryPolicy(max_attempts=5, base_delay=0), br, sleep=lambda s: None)
    assert br.state == "open"
    cm = CheckpointManager(tmp_path / "ck", save_total_limit=2)
    for step, loss in ((1, 3.0), (2, 1.0), (3, 2.0), (4, 2.5)):
        cm.save(step, lambda d: (d / "x.txt").write_text("x"), {"eval_loss": loss})
    names = [p.name for p in cm.list()]
    assert "checkpoint-2" in names and "checkpoint-4" in names and "checkpoint-1" not in names   # best is kept
    assert cm.latest().name == "checkpoint-4" and cm.best().name == "checkpoint-2"


def test_registry_graph_and_hf_conversion():
    from transformers import LlamaConfig as HC, LlamaForCausalLM as HM
    from trainscale_b200.registry import DependencyGraph, KernelCapabilityMatrix, DEFAULT_CONTRACTS, RegistryValidator, detect_capabilities, patch_model
    g = DependencyGraph()
    g.add("a", ["b"])
    g.add("b", ["c"])
    assert g.topological_order() == ["c", "b", "a"]
    g.add("c", ["a"])
    assert g.find_cycles() and pytest.raises(ValueError, g.topological_order)
    m = KernelCapabilityMatrix(DEFAULT_CONTRACTS)
    assert RegistryValidator(m).validate() == []
    assert m.resolve("flash_attention_tcgen05", detect_capabilities()) in ("flash_attention_tcgen05", "attention_torch")
    hf = HM(HC(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, max_position_embeddings=64)).eval()
    mine = patch_model(hf, dtype=torch.float32).eval()
    ids = torch.randint(0, 256, (2, 12))
    assert (mine(ids).logits - hf(ids).logits).abs().max() < 1e-4
    assert abs(mine(ids, labels=ids).loss.item() - hf(ids, labels=ids).loss.item()) < 1e-5


def test_lora_quant_rl_metrics():
    from trainscale_b200.lora import count_trainable, get_peft_model, merge_and_unload
    from trainscale_b200.models.llama import build_model
    from trainscale_b200.quantization import block_dequantize_fp8, block_quantize_fp8, fast_dequantize, quantize_nf4
    from trainscale_b200.rl import compute_advantages, grpo_loss, left_pack_padding, selective_log_softmax
    from trainscale_b200.metrics import BLEU, F1Score, LossTracker, Perplexity
    m = build_model("tiny", dtype=torch.float32, seed=0)
    ids = torch.randint(0, 32000, (1, 8))
    base = m(ids).logits
    get_peft_model(m, r=4, target_modules=["q_proj", "v_proj"])
    t, tot = count_trainable(m)
    assert 0 < t < 0.01 * tot and torch.allclose(m(ids).logits, base, atol=1e-5)
    for n, p in m.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    tuned = m(ids).logits
    merge_and_unload(m)
    assert (m(ids).logits - tuned).abs().max() < 1e-4 and not any("lora_" in n for n, _ in m.named_parameters())
    w = torch.randn(200, 130)
    q, s = block_quantize_fp8(w)
    assert (block_dequantize_fp8(q, s, dtype=torch.float32) - w).abs().max() < 0.3 and s.shape == (2, 2)
    pk, am, sh = quantize_nf4(w)
    assert (fast_dequantize(pk, am, sh, torch.float32) - w).abs().mean() < 0.15
    lg, idx = torch.randn(3, 7), torch.tensor([1, 2, 3])
    assert torch.allclose(selective_log_softmax(lg, idx), torch.log_softmax(lg, -1).gather(1, idx[:, None]).squeeze(1), atol=1e-6)
    adv = compute_advantages(torch.tensor([1.0, 2, 3, 4]), 4)
    assert abs(float(adv.mean())) < 1e-6
    lp = torch.zeros(4, 3)
    assert float(grpo_loss(lp, lp, lp, adv, torch.ones(4, 3))) == pytest.approx(0.0, abs=1e-6)
    ids2, mk = left_pack_padding(torch.tensor([[0, 5, 0, 6]]), torch.tensor([[0, 1, 0, 1]]))
    assert ids2.tolist() == [[5, 6, 0, 0]]
    f = F1Score()
    f.update(torch.tensor([0, 1, 1]), torch.tensor([0, 1, 0]))
    assert 0 < f.compute() < 1
    b = BLEU()
    b.update(["a b c d e"], ["a b c d e"])
    assert b.compute() == pytest.approx(1.0)
    p = Perplexity()
    p.update(torch.zeros(4, 10), torch.zeros(4, dtype=torch.long))
    assert p.compute() == pytest.approx(10.0, rel=1e-4)
    lt = LossTracker()
    lt.update(2.0, 10)
    lt.update(4.0, 30)
    assert lt.mean == pytest.approx(3.5)


def test_ptrr_balancer_and_planning_helpers():
    import torch
    from trainscale_b200.parallel import cp, mesh
    bal = [cp.create_balancer("ptrr", 4, r) for r in range(4)]
    idx = torch.cat([b.indices(64) for b in bal]).sort().values
    assert torch.equal(idx, torch.arange(64))
    assert bal[1].indices(64)[:4].tolist() == [4, 5, 6, 7] and bal[1].indices(64)[4:8].tolist() == [24, 25, 26, 27]
    x = torch.arange(64).view(1, 64)
    assert torch.equal(bal[0].unshard([b.shard(x) for b in bal]), x)
    est = mesh.MemoryEstimator.estimate_per_gpu_memory
    one = est(8_030_000_000, 1, 8192, 4096, 32, intermediate_dim=14336)
    eight = est(8_030_000_000, 1, 8192, 4096, 32, dp_shard_degree=8, intermediate_dim=14336)
    assert one > eight and mesh.MemoryEstimator.fits(eight) and not mesh.MemoryEstimator.fits(one, capacity_gb=80)
    sel = mesh.CommAlgorithmSelector(8)
    assert sel.all_reduce(4096) == "one_shot_p2p" and sel.all_reduce(1 << 28) == "multimem"
    assert mesh.CommAlgorithmSelector(8, nvswitch=False).all_reduce(1 << 28) == "ring"
    assert mesh.HardwareDetector.detect()["num_gpus"] >= 0


def test_gradient_plumbing_helpers_single_process():
    import torch
    from trainscale_b200.parallel import dist_utils
    out = torch.zeros(4)
    dist_utils.reduce_scatter_with_fp32_accumulation(out, torch.arange(4.0))
    assert out.tolist() == [0.0, 1.0, 2.0, 3.0]
    lin = torch.nn.Linear(4, 4)
    lin(torch.ones(2, 4)).sum().backward()
    g0 = lin.weight.grad.clone()
    dist_utils.finalize_model_grads(lin, num_tokens=torch.tensor(4.0), dp_group=False)
    assert torch.allclose(lin.weight.grad, g0 / 4)
    mgr = dist_utils.DistributedManager()
    assert mgr is dist_utils.DistributedManager() and mgr.world_size == 1
    assert mgr.reduce_dict({"loss": 2.0}) == {"loss": 2.0}
    sync = dist_utils.GradientSynchronizer(engine=object(), accumulation_steps=4)
    assert [sync.should_sync(i) for i in range(4)] == [False, False, False, True]


def test_sophia_hutchinson_hessian_diagonal():
    import torch
    from trainscale_b200.optim import SophiaG
    d = torch.tensor([1.0, 2.0, 3.0, 4.0])
    x = torch.randn(4, requires_grad=True)
    opt = SophiaG([x], betas=(0.9, 0.5))
    opt.update_hessian_hutchinson(0.5 * (d * x * x).sum())          # diagonal Hessian: u * (H u) = d exactly
    torch.testing.assert_close(opt.state[x]["h"], 0.5 * d)
    x.grad = torch.ones(4)
    before = x.detach().clone()
    opt.step()
    assert not torch.equal(before, x.detach())


def test_adapter_save_load_and_attention_interface(tmp_path):
    import json
    import pytest
    import torch
    from trainscale_b200.lora import get_peft_model, load_adapter, lora_state_dict, save_adapter
    from trainscale_b200.models.llama import LlamaConfig, build_model
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16)
    m = build_model(cfg, dtype=torch.float32, device="cpu", seed=0)
    get_peft_model(m, r=4)
    for n, p in m.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p)
    save_adapter(m, tmp_path)
    keys = json.loads((tmp_path / "adapter_config.json").read_text())["target_modules"]
    assert "q_proj" in keys and "down_proj" in keys
    m2 = build_model(cfg, dtype=torch.float32, device="cpu", seed=0)
    get_peft_model(m2, r=4)
    assert load_adapter(m2, tmp_path) == []
    a, b = lora_state_dict(m), lora_state_dict(m2)
    assert len(a) == 28 and all(torch.equal(a[k], b[k]) for k in a)
    ids = torch.randint(0, 128, (1, 12))
    torch.testing.assert_close(m(ids).logits, m2(ids).logits)
    # HF model routed through the registered attention function: unchanged results on CPU (falls back to SDPA)
    transformers = pytest.importorskip("transformers")
    from trainscale_b200.registry import ModelInfo, ModelMeta, auto_patch_attention
    hf = transformers.LlamaForCausalLM(transformers.LlamaConfig(
        vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2)).eval()
    with torch.no_grad():
        ref = hf(ids).logits
        assert auto_patch_attention(hf) == 2 and hf.config._attn_implementation == "trainscale_flash"
        torch.testing.assert_close(hf(ids).logits, ref)
    assert ModelMeta is ModelInfo
    from trainscale_b200.utils.cuda_graphs import CUDAGraphManager, compilation_debug_mode, get_compilation_stats
    mg = CUDAGraphManager()
    before = get_compilation_stats()["eager_calls"]
    with compilation_debug_mode(log=lambda s: None):
        assert float(mg.run(lambda x: x + 1, torch.ones(2))[0]) == 2.0
    assert get_compilation_stats()["eager_calls"] == before + 1 and get_compilation_stats(mg)["signatures"] == 0


def test_tracing_utilities(tmp_path):
    import torch
    from trainscale_b200.utils import tracing as T
    timer = T.PhaseTimer("cpu")
    for _ in range(2):
        with timer("forward"):
            torch.randn(8, 8) @ torch.randn(8, 8)
    s = timer.summary()
    assert s["forward"]["count"] == 2 and s["forward"]["total_ms"] >= 0
    T.enable_nvtx(True)
    with T.nvtx_range("phase"):          # without a GPU the range is a no-op, with one it pushes / pops
        pass
    T.nvtx_mark("tick")
    T.enable_nvtx(False)
    with T.profile_steps(tmp_path, wait=0, warmup=1, active=2) as prof:
        for _ in range(4):
            torch.randn(32, 32) @ torch.randn(32, 32)
            prof.step()
    assert (tmp_path / "trace_0.json").stat().st_size > 0


def test_qwen2_bias_and_mixtral_moe_decoders_match_huggingface():
    import pytest
    import torch
    transformers = pytest.importorskip("transformers")
    from trainscale_b200.models.llama import build_model, preset_config
    from trainscale_b200.registry import patch_model
    torch.manual_seed(0)
    ids = torch.randint(0, 64, (2, 12))
    kw = dict(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2)
    cases = (transformers.MixtralForCausalLM(transformers.MixtralConfig(num_local_experts=4, num_experts_per_tok=2,
                                                                         sliding_window=None, **kw)),
             transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**kw)),
             transformers.GemmaForCausalLM(transformers.GemmaConfig(head_dim=16, **kw)))
    for hf in cases:
        hf = hf.eval()
        with torch.no_grad():
            for n, p in hf.named_parameters():
                if n.endswith("bias") or (type(hf).__name__.startswith("Gemma") and "norm" in n):
                    p.normal_(0, 0.5)
            ref = hf(ids).logits
            m = patch_model(hf, dtype=torch.float32, device="cpu").eval()
            torch.testing.assert_close(m(ids).logits, ref, rtol=1e-5, atol=1e-6)
            back = type(hf)(hf.config).eval()
            missing = back.load_state_dict(m.to_hf_state_dict(), strict=False).missing_keys
            assert [k for k in missing if k != "lm_head.weight"] == []          # a tied head has no tensor of its own
            torch.testing.assert_close(back(ids).logits, ref)
    # a mixture-of-experts model trains through the ordinary path (router and biases receive gradients, balance loss on)
    cfg = preset_config("moe-tiny", vocab_size=128, router_aux_loss_coef=0.01, attention_bias=True)
    m = build_model(cfg, dtype=torch.float32, device="cpu", seed=0)
    assert m.num_parameters() == cfg.num_parameters()
    ids = torch.randint(0, 128, (2, 16))
    base = m(ids, labels=ids).loss
    base.backward()
    assert float(m.model.layers[0].mlp.router.grad.abs().sum()) > 0
    assert float(m.model.layers[0].self_attn.bqkv.grad.abs().sum()) > 0
    m.eval()
    assert float(m(ids, labels=ids).loss) < float(base)            # no balance term outside training
    assert m.hf_config_dict()["model_type"] == "mixtral"


@pytest.mark.parametrize("name", ["adamw", "adam8bit", "lion", "lamb", "adafactor", "came", "sophia", "prodigy",
                                  "schedule_free", "muon", "adopt"])
def test_every_optimizer_of_the_zoo_reduces_a_least_squares_loss(name):
    """Each optimizer behind `create_optimizer`, on its PyTorch path (no GPU): 150 steps on a small regression cut the
    loss at least in half and keep the weights finite."""
    from trainscale_b200.optim import create_optimizer
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(32, 16) * 0.1)
    b = torch.nn.Parameter(torch.zeros(16))
    x = torch.randn(128, 32)
    y = x @ torch.randn(32, 16)
    lr = {"lion": 3e-3, "prodigy": 1.0, "sophia": 1e-2, "muon": 2e-2, "lamb": 2e-2}.get(name, 1e-2)
    opt = create_optimizer([w, b], name=name, lr=lr, weight_decay=0.0)
    if hasattr(opt, "train"):
        opt.train()
    first = None
    for i in range(150):
        loss = ((x @ w + b - y) ** 2).mean()
        first = loss.item() if first is None else first
        opt.zero_grad()
        loss.backward()
        if name == "sophia" and i % 10 == 0:
            opt.update_hessian()
        opt.step()
    if hasattr(opt, "eval"):
        opt.eval()
    last = ((x @ w + b - y) ** 2).mean().item()
    # AdaFactor's relative step (1e-2 x RMS of the weights) is slow by construction on weights this small
    bound = 0.8 if name == "adafactor" else 0.5
    assert bool(torch.isfinite(w).all()) and last < bound * first, (name, first, last)


def test_ranking_segmentation_and_distillation_losses_against_direct_formulas():
    """The losses of losses/extra.py against loop-form restatements of their definitions."""
    import math

    import torch
    import torch.nn.functional as F

    from trainscale_b200 import losses as L
    torch.manual_seed(0)
    scores, rel = torch.randn(3, 6, requires_grad=True), torch.randint(0, 4, (3, 6)).float()
    # ListMLE: -sum_i log softmax over the remaining items, in ideal order
    want = 0.0
    for b in range(3):
        order = sorted(range(6), key=lambda i: (-rel[b, i].item(), i))
        s = scores[b, order]
        want += -sum(s[i] - torch.logsumexp(s[i:], 0) for i in range(6))
    got = L.ListMLELoss()(scores, rel)
    assert abs(float(got) - float(want) / 3) < 1e-5
    got.backward()
    assert scores.grad.abs().sum() > 0
    # LambdaRank: pair loop
    ranks = scores.detach().argsort(1, descending=True).argsort(1)
    tot = 0.0
    for b in range(3):
        gains = 2.0 ** rel[b] - 1
        disc = 1 / torch.log2(ranks[b].float() + 2)
        idcg = (gains.sort(descending=True).values / torch.log2(torch.arange(6).float() + 2)).sum().clamp(min=1e-8)
        acc = 0.0
        for i in range(6):
            for j in range(i + 1, 6):
                d = abs(gains[i] * (disc[j] - disc[i]) + gains[j] * (disc[i] - disc[j])) / idcg
                sgn = math.copysign(1.0, rel[b, i] - rel[b, j]) if rel[b, i] != rel[b, j] else 0.0
                acc += d * math.log1p(math.exp(-sgn * float(scores[b, i] - scores[b, j])))
        tot += acc / 15
    assert abs(float(L.LambdaRankLoss()(scores.detach(), rel)) - float(tot) / 3) < 1e-5
    # segmentation
    p, t = torch.rand(2, 3, 4, 4), (torch.rand(2, 3, 4, 4) > 0.5).float()
    inter = (p * t).flatten(2).sum(-1)
    union = p.flatten(2).sum(-1) + t.flatten(2).sum(-1) - inter
    assert torch.allclose(L.IoULoss()(p, t), (1 - (inter + 1) / (union + 1)).mean())
    fp, fn = (p * (1 - t)).flatten(2).sum(-1), ((1 - p) * t).flatten(2).sum(-1)
    tv = (inter + 1) / (inter + 0.7 * fp + 0.3 * fn + 1)
    assert torch.allclose(L.FocalTverskyLoss()(p, t), ((1 - tv) ** 0.75).mean())
    assert torch.allclose(L.BoundaryLoss()(p, t - 0.5), (p * (t - 0.5)).sum((2, 3)).mean())
    assert torch.allclose(L.CharbonnierLoss(1e-3)(p, t), torch.sqrt((p - t) ** 2 + 1e-6).mean())
    # GHM-C: with one bin every weight is 1, so the loss is plain cross-entropy; with many bins it is a reweighting
    logits, y = torch.randn(32, 5), torch.randint(0, 5, (32,))
    assert torch.allclose(L.GHMCLoss(bins=1)(logits, y), F.cross_entropy(logits, y), atol=1e-6)
    g = 1 - F.softmax(logits, 1).gather(1, y[:, None]).squeeze(1)
    idx = (g * 10).floor().clamp(max=9).long()
    w = 32 / (torch.bincount(idx, minlength=10).clamp(min=1).float() * 10)
    assert torch.allclose(L.GHMCLoss(bins=10)(logits, y), (F.cross_entropy(logits, y, reduction="none") * w[idx]).mean(),
                          atol=1e-6)
    yb = (torch.rand(32) > 0.5).float()
    assert torch.isfinite(L.GHMCLoss(bins=5, momentum=0.5)(logits[:, 0], yb, mask=torch.rand(32) > 0.2))
    # distillation
    s, tt = torch.randn(2, 7, 16), torch.randn(2, 7, 24)
    fd = L.FeatureDistillationLoss("cosine")
    assert fd(s, tt).shape == () and fd.projection.weight.shape == (24, 16)
    a, b = torch.randn(2, 2, 5, 5), torch.randn(2, 2, 5, 5)
    kl = L.AttentionDistillationLoss("kl", 2.0)(a, b)
    want = F.kl_div(F.log_softmax(a.reshape(-1, 5) / 2, -1), F.softmax(b.reshape(-1, 5) / 2, -1), reduction="batchmean")
    assert torch.allclose(kl, want)
    pl = L.PerceptualLoss(torch.nn.Conv2d(3, 4, 3), normalize=False)
    assert float(pl(p, p)) == 0.0 and float(pl(p, t)) > 0
    m = L.create_label_smoothing_matrix(10, 0.1)
    assert m.shape == (10, 10) and abs(float(m[3, 3]) - 0.9) < 1e-6 and abs(float(m[3, 4]) - 0.01) < 1e-6
    out = L.LossOutput(torch.tensor(1.0), {"ppl": 2.7})
    assert out.aux_loss is None and L.create_loss("iou").__class__ is L.IoULoss


def test_checkpoint_catalogue_contracts_and_layer_patches():
    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    from trainscale_b200 import registry as R
    n = R.register_llama_models()
    assert n > 0 and R.register_llama_models() == 0                       # idempotent
    info = R.get_checkpoint_info("meta-llama/Llama-3.1-8B-Instruct")
    assert isinstance(info, R.LlamaModelInfo) and info.mlp_class == "LlamaMLP" and info.model_path.endswith("Instruct")
    assert R.get_checkpoint_info("unsloth/Llama-3.1-8B-Instruct-bnb-4bit").quant_type is R.QuantType.BNB_4BIT
    total = R.register_all_models()
    assert total > 100 and len(R.CHECKPOINT_REGISTRY) == n + total
    assert all(i.is_multimodal for i in R.search_models(is_multimodal=True)) and R.search_models(is_multimodal=True)
    assert {i.size for i in R.search_models(base_name="gemma", quant_type=R.QuantType.NONE, org="google")} >= {"2", "9", "27"}
    assert R.register_model(R.CheckpointInfo, "me", "Tiny", "1", "0.1").model_path == "me/Tiny-1-0.1B"
    assert R.register_model(R.CheckpointInfo, "me", "Tiny", "1", "0.1") is None
    assert R.CheckpointInfo.construct_model_name("DeepSeek", "V3", "default", R.QuantType.BF16, "Chat") == "DeepSeek-V3-Chat-bf16"

    # contracts
    c = R.BaseModuleContract("needs_tcgen05", _hardware_requirements=frozenset({R.Capability.TCGEN05}),
                             _dependencies=frozenset({"gemm_tcgen05", "nowhere"}))
    cpu = R.HardwareCapability("cpu", (0, 0), 0, 0.0, frozenset())
    errs = c.validate(cpu, known={"gemm_tcgen05"})
    assert [type(e) for e in errs] == [R.HardwareError, R.DependencyError] and errs[1].missing_deps == ("nowhere",)
    b200 = R.HardwareCapability("b200", (10, 0), 148, 180.0, frozenset({R.Capability.TCGEN05}))
    assert c.validate(b200) == [] and c.to_contract().requires == (R.Capability.TCGEN05,)
    assert R.get_registry_validator() is R.get_registry_validator() and R.get_registry_validator().validate() == []

    @R.requires_capability(R.Capability.TCGEN05)
    def only_on_blackwell():
        return 1
    if not R.has_capability(R.Capability.TCGEN05):
        import pytest
        with pytest.raises(RuntimeError, match="TCGEN05"):
            only_on_blackwell()

    # layer patches by class name
    class GemmaMLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = nn.Linear(8, 16, bias=False), nn.Linear(8, 16, bias=False), nn.Linear(16, 8, bias=False)

        def forward(self, x):
            raise AssertionError("the patched forward must run")
    net = nn.Sequential(GemmaMLP())
    assert R.apply_layer_patches(net) == ["0"]
    x = torch.randn(3, 8)
    m = net[0]
    want = m.down_proj(F.gelu(m.gate_proj(x), approximate="tanh") * m.up_proj(x))
    assert torch.allclose(net(x), want, atol=1e-5)


def test_optimizer_helpers_core_records_and_presets():
    import os

    import pytest
    import torch

    from trainscale_b200 import optim as O
    from trainscale_b200.config import sota_config as S
    from trainscale_b200.config import training_args as T
    from trainscale_b200.core.errors import DeviceNotAvailableError, EarlyStoppingError, TrainingLoopError
    from trainscale_b200.core.types import CheckpointStrategy, GradientInfo, StepMetrics, WarmupType
    m = torch.nn.Linear(256, 256)
    m(torch.randn(4, 256)).sum().backward()
    total, mx, mn = O.compute_grad_norm(m.parameters())
    want = torch.sqrt(m.weight.grad.pow(2).sum() + m.bias.grad.pow(2).sum())
    assert abs(total - float(want)) < 1e-2 and mx >= mn > 0
    info = O.clip_grad_value_(m.parameters(), 0.01)
    assert isinstance(info, GradientInfo) and info.clipped and float(m.weight.grad.abs().max()) <= 0.01
    opt = O.create_adafactor_for_llm(m.parameters(), "70b")
    opt.step()
    assert opt.param_groups[0]["clip_threshold"] == 0.5
    fp = O.get_optimizer_memory_footprint(opt)
    assert fp["compression_ratio"] > 50 and fp["total_bytes"] > 0          # factored moments: rows + columns
    assert O.check_optimizer_compatibility(opt, m)["is_compatible"]
    extra = torch.nn.Linear(2, 2)
    bad = O.check_optimizer_compatibility(opt, torch.nn.Sequential(m, extra))
    assert not bad["is_compatible"] and any("not in the optimizer" in w for w in bad["warnings"])
    assert O.determine_factorization((4096, 4096)) is O.FactorizationMode.BLOCK
    assert O.determine_factorization((512, 512)) is O.FactorizationMode.ROW_COL
    assert O.determine_factorization((64, 4096)) is O.FactorizationMode.NONE
    assert O.compute_rho_jit(0, -0.8) == 0.0 and O.compute_rho_jit(10 ** 6, -0.8) == 0.999
    assert abs(O.compute_rms_jit(torch.full((10,), 3.0)) - 3.0) < 1e-6

    class SignSGD(O.BaseOptimizer):
        def __init__(self, params, lr=0.1):
            super().__init__(params, dict(lr=lr, max_grad_norm=1.0))

        def _update(self, p, g, st, grp):
            p.add_(g.sign(), alpha=-grp["lr"])
    w0 = m.weight.detach().clone()
    o2 = SignSGD(m.parameters())
    o2.step()
    assert abs(float((m.weight - w0).abs().max()) - 0.1) < 1e-6 and o2.metrics.total_steps == 1
    assert o2.lifecycle is O.OptimizerState.STEPPED and o2.state[m.weight]["step"] == 1
    k = O.KahanAccumulator()
    for _ in range(10):
        k.add(0.1)
    assert k.value == 1.0
    st = O.AdaFactorState((8, 16), "cpu", torch.float32, True, True).initialize()
    assert st.memory_bytes() == (8 + 16 + 128) * 4 and st.snapshot().exp_avg_sq is None
    assert O.AdaFactorConfig(lr=1e-3, relative_step=False).build(m.parameters()).defaults["lr"] == 1e-3
    assert O.create_lamb(m.parameters(), max_trust_ratio=5.0).defaults["clamp_trust"] == (0.0, 5.0)
    assert O.create_adamw(m.parameters(), max_grad_norm=1.0).max_grad_norm == 1.0 and O.get_triton_version() is None
    x = torch.randn(3, 5)
    assert torch.allclose(O.stable_softmax(x), torch.softmax(x, -1), atol=1e-6)

    e = EarlyStoppingError(metric_name="loss", metric_value=1.0, patience=3)
    assert isinstance(e, TrainingLoopError) and e.patience == 3 and "patience=3" in str(e)
    assert DeviceNotAvailableError("no gpu", "cuda", ("cpu",)).available_devices == ("cpu",)
    assert WarmupType("linear") is WarmupType.LINEAR and CheckpointStrategy.BEST_AND_LAST.value == "best_and_last"
    assert StepMetrics(1.0, 1e-4, 0.5, 1e4, 100.0, 12.0).component_losses is None

    c = S.get_dpo_preset("m")
    assert c.loss.type is S.LossType.DPO and c.rl.algorithm is S.RLAlgorithm.DPO and c.rl.enabled
    assert S.get_export_gguf_preset("/o", "q8_0").format is S.ExportFormat.GGUF_Q8
    with pytest.raises(ValueError):
        S.get_export_gguf_preset("/o", "q3")
    assert T.get_qlora_config("m", r=8).lora_alpha == 16 and T.get_pretraining_config("m").pack_sequences
    assert T.get_full_finetune_config("m").to_sota_dict()["optimizer"]["learning_rate"] == 1e-5
    os.environ["TS_TEST_OUT"] = "/tmp/ts_x"
    assert T.load_training_config_from_dict({"output_dir": "${TS_TEST_OUT}"}).output_dir == "/tmp/ts_x"
    with pytest.raises(ValueError, match="learning_rate"):
        T.load_training_config_from_dict({"learning_rate": "abc"})


def test_inference_hub_and_introspection_reference_names(tmp_path):
    import torch

    from trainscale_b200 import hub as H
    from trainscale_b200 import introspection as I
    from trainscale_b200.inference import engine as E
    cfg = E.EngineConfig(model="tiny", device="cpu", dtype="float32")
    probe = E.HardwareProbe.probe()
    assert probe["gpu_count"] == len(probe["devices"]) and "recommended_attention" in probe
    out = E.run_batch_demo(cfg, ["hello", "abc"], E.GenerationParams(max_tokens=3, temperature=0.0))
    assert len(out) == 2 and all(r.metrics.completion_tokens == 3 for r in out)
    eng = E.SOTAInferenceEngine(cfg)
    assert E.ResultStatus.of(eng.generate("x", E.GenerationParams(max_tokens=2))) is E.ResultStatus.OK
    assert E.ResultStatus.of(eng.generate("x", E.GenerationParams(max_tokens=0))) is E.ResultStatus.ERR
    req = E.InferenceRequest("hi", params=E.GenerationParams(max_tokens=2, temperature=0.0))
    queued = req.submit(eng)
    while eng.core.has_unfinished():
        eng.core.step()
    assert len(queued.output_ids) == 2 and req.metrics is queued.metrics and len(req.request_id) == 32
    assert E.run_benchmark(cfg, 2, 8, 4)["output_tokens_per_second"] > 0
    assert E.SchedulerPolicy("fcfs") is E.SchedulerPolicy.FCFS and E.QuantizationMethod.FP8.value == "fp8"
    assert E.ParallelStrategy.TENSOR.value == "tensor"

    hc = H.HubConfig(shard_size_bytes=4096, repo_id="me/x", token="t")
    hc.serializer().save({"a": torch.randn(32, 32), "b": torch.randn(32, 32), "c": torch.randn(8)}, tmp_path / "m")
    res = H.SerializationResult.describe(tmp_path / "m")
    assert len(res.shards) == 3 and res.format == "safetensors" and res.shards[0].tensor_names == ("a",)
    assert res.total_bytes == sum(s.byte_size for s in res.shards) and res.shards[1].byte_offset == res.shards[0].byte_size
    assert hc.manager().repo_id == "me/x" and hc.manager().policy.max_attempts == 3
    cm = H.CheckpointManager(tmp_path / "ck")
    p = cm.save(5, lambda t: (t / "x").write_text("1"), {"loss": 1.5, "epoch": 2})
    meta = H.CheckpointMetadata.read(p)
    assert (meta.step, meta.epoch, meta.loss) == (5, 2, 1.5) and len(meta.sha256) == 64 and meta.path == p
    b = H.CircuitBreaker(failure_threshold=1)
    assert H.CircuitState.of(b) is H.CircuitState.CLOSED
    b.record_failure()
    assert H.CircuitState.of(b) is H.CircuitState.OPEN
    assert H.classify_hub_error(TimeoutError()) is H.HubErrorCode.TIMEOUT
    assert H.classify_hub_error(ConnectionError()) in H.RETRIABLE and H.classify_hub_error(ValueError()) not in H.RETRIABLE
    g = H.HubMetrics()
    g.record_upload(10, 2_000_000, True)
    g.record_upload(10, 4_000_000, False)
    g.record_retry()
    s = g.summary()
    assert (s["uploads_total"], s["uploads_failed"], s["bytes_uploaded"], s["retries_total"]) == (2, 1, 10, 1)
    assert H.get_hub_metrics() is H.get_hub_metrics()

    rows = {"train": [{"question": "q", "answer": "a", "tags": ["x"], "meta": {"k": 1}}], "test": []}
    md = I.discover_dataset(rows).unwrap()
    assert I.get_default_split(rows).unwrap() == "train" and I.get_default_split(md).unwrap() == "train"
    assert I.describe_dataset(md)[0].splits[0] == I.SplitInfo("train", 1)
    feats = {f.name: f for f in I.describe_features(rows["train"])}
    assert feats["tags"].is_list and feats["meta"].is_nested and not feats["question"].is_list
    assert I.fuzzy_match_columns(["question", "answer", "Txt"], ["prompt", "completion", "text"]).unwrap() == \
        {"prompt": "question", "completion": "answer", "text": "Txt"}
    kinds = [m.match_type for m in I.match_columns(["question", "answr", "text"], ["prompt", "answer", "text"])]
    assert kinds == ["pattern", "fuzzy", "exact"]
    assert I.fuzzy_match_columns(["a"], ["prompt"]).is_err()
    assert I.fuzzy_match_columns(["a"], ["prompt"], {"prompt": "a"}).unwrap() == {"prompt": "a"}
    assert abs(I.normalized_similarity("Prompt", "prompts") - 6 / 7) < 1e-9 and I.get_introspector() is I.get_introspector()


def test_training_trackers_full_surface():
    import math
    import time

    import torch

    from trainscale_b200.metrics import (AccuracyTracker, GradientTracker, LossTracker, ThroughputTracker,
                                         TrainingMetrics, create_training_metrics)
    lt = LossTracker()
    lt.update(2.0, num_tokens=10, num_samples=2)
    lt.update(1.0, num_tokens=30, accumulation_steps=4)          # the loss had been divided by 4
    assert lt.compute_avg() == (2.0 * 10 + 4.0 * 30) / 40 and lt.last_loss == 4.0 and lt.step_count == 2
    assert lt.total_tokens == 40 and lt.total_samples == 3 and lt.get_history(1) == [4.0]
    assert abs(lt.compute_ema() - (0.99 * 2.0 + 0.01 * 4.0)) < 1e-12 and lt.compute_variance() == 2.0
    assert abs(lt.compute_ppl() - math.exp(3.5)) < 1e-9 and lt.sync() == 3.5
    logits, labels = torch.randn(2, 5, 7), torch.randint(0, 7, (2, 5))
    labels[0, 1] = -100
    want = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 7), labels[:, 1:].reshape(-1), ignore_index=-100)
    lt2 = LossTracker()
    assert abs(lt2.update_from_logits(logits, labels) - float(want)) < 1e-5 and lt2.total_tokens == 7
    sd = lt.state_dict()
    lt3 = LossTracker()
    lt3.load_state_dict(sd)
    assert lt3.compute_avg() == 3.5 and lt3.step_count == 2
    lt.reset()
    assert lt.total_tokens == 0 and lt.compute_avg() == 0.0

    acc = AccuracyTracker()
    a = acc.update_from_logits(logits, labels)
    pred = logits[:, :-1].argmax(-1)
    m = labels[:, 1:] != -100
    assert acc.total == 7 and abs(a - float(((pred == labels[:, 1:]) & m).sum()) / 7) < 1e-9
    acc.update(3, 3)
    assert acc.total == 10 and acc.sync() == acc.compute() == acc.accuracy

    net = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    net(torch.randn(5, 4)).sum().backward()
    gt = GradientTracker(max_norm=1e-3)
    n = gt.update(net.parameters())
    want = math.sqrt(sum(float(p.grad.pow(2).sum()) for p in net.parameters()))
    assert abs(n - want) < 1e-5 and gt.compute_norm() == n and gt.is_anomaly() and not gt.has_nan_or_inf()
    allg = torch.cat([p.grad.reshape(-1) for p in net.parameters()])
    assert abs(gt.compute_mean() - float(allg.mean())) < 1e-6 and abs(gt.compute_std() - float(allg.std(unbiased=False))) < 1e-5
    gt.update_from_model(net)
    top = gt.get_top_layers(2)
    assert len(gt.get_layer_norms()) == 4 and top[0][1] >= top[1][1] and gt.step_count == 2
    net[0].weight.grad[0, 0] = float("nan")
    gt.update(net)
    assert gt.has_nan() and not gt.has_inf() and gt.nan_count == 1
    gt.update(0.5)                                                  # a norm computed elsewhere
    assert gt.compute_norm() == 0.5 and set(gt.histogram()) == {"p10", "p25", "p50", "p75", "p90", "max"}
    assert "gradient/norm_ema" in gt.log_dict()
    g2 = GradientTracker()
    g2.load_state_dict(gt.state_dict())
    assert g2.step_count == gt.step_count and abs(g2.compute_ema_norm() - gt.compute_ema_norm()) < 1e-12

    tt = ThroughputTracker(flops_per_token=6e3, peak_tflops=1e-6, use_cuda_events=False)
    tt.start()
    time.sleep(0.02)
    tt.update(samples=2, tokens=1000)
    time.sleep(0.02)
    tt.update(samples=2, tokens=1000)
    assert tt.total_tokens == 2000 and tt.total_samples == 4 and tt.step_count == 2 and tt.elapsed_seconds() >= 0.04
    assert 0 < tt.tokens_per_sec() < 1e5 and tt.samples_per_sec() > 0 and tt.tokens_per_sec_window() > 0
    assert abs(tt.compute_tflops() / (tt.tokens_per_sec() * 6e3 / 1e12) - 1) < 0.05 and tt.compute_mfu() > 0   # the clock runs
    assert tt.compute_mfu(model_params=1000) > 0 and "throughput/mfu" in tt.log_dict()
    tt.sync()
    tt.reset()
    assert tt.total_tokens == 0 and tt.step_count == 0

    tm = create_training_metrics(model=net, log_prefix="train")
    assert tm.model_params == sum(p.numel() for p in net.parameters())
    tm.start()
    tm.new_epoch(1)
    time.sleep(0.01)
    tm.update_step(torch.tensor(2.0), logits=logits, labels=labels, batch_size=2, num_tokens=8, lr=1e-4, grad_norm=0.7)
    tm.update_step(1.0, model=net, batch_size=2, num_tokens=8)
    out = tm.compute()
    assert out["global_step"] == 2 and out["epoch"] == 1 and out["loss"] == 1.5 and out["lr"] == 1e-4
    assert out["total_tokens"] == 16 and 0.0 <= out["accuracy"] <= 1.0
    assert set(tm.log_dict()) >= {"train/loss", "train/ppl", "train/step", "train/mfu"}
    assert tm.format_log_string().startswith("step=2 | loss=1.5000 | ppl=")
    tm2 = TrainingMetrics()
    tm2.load_state_dict(tm.state_dict())
    assert tm2.compute(sync=False)["global_step"] == 2 and "tokens_per_second" in tm.summary()
    tm.reset()
    assert tm.loss.total_tokens == 0 and tm.compute()["global_step"] == 2
    tm.reset_all()
    assert tm.compute()["global_step"] == 0
