"""The reference's class-level API of the distributed layer (FSDP2 facade, general pipeline API) on CPU."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.nn as nn

CASES = Path(__file__).parent / "dist_cases"


def launch(case, nproc, port, *args, timeout=300):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(CASES / case), *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)


def test_fsdp2_facade_two_ranks():
    r = launch("fsdp2_facade.py", 2, 29681)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT ok=True" in r.stdout


def test_fsdp2_config_and_helpers():
    from trainscale_b200.parallel import fsdp2 as F
    c = F.FSDP2Config(sharding_strategy="hybrid_shard", mixed_precision="bf16", bucket_size_mb=40)
    assert c.sharding_strategy is F.ShardingStrategy.HYBRID_SHARD and c.bucket_size_bytes == 40 * 2 ** 20
    assert c.to_engine_config().sharding_strategy == "FULL_SHARD"
    assert F.ShardingStrategy.NO_SHARD.requires_all_gather is False
    assert F.MixedPrecisionPolicy.FULL_BF16.get_param_dtype() is torch.bfloat16
    with pytest.raises(ValueError):
        F.FSDP2Config(gradient_accumulation_steps=0)
    with pytest.raises(ValueError):
        F.FSDP2Config(mixed_precision="fp16")
    pool = F.MemoryPool("cpu")
    a = pool.allocate(1000, torch.float32)
    ptr = a.data_ptr()
    pool.release(a)
    b = pool.allocate(900, torch.float32)
    assert b.data_ptr() == ptr and pool.get_stats()["hits"] == 1
    acc = F.GradientAccumulator(2)
    lin = nn.Linear(4, 4)
    for _ in range(2):
        lin(torch.ones(1, 4)).sum().backward()
        acc.accumulate(lin)
    assert acc.should_sync
    acc.apply_to_model(lin)
    assert torch.allclose(lin.weight.grad, torch.ones(4, 4))
    mc = F.MetricsCollector("cpu")
    with mc.measure_forward():
        pass
    mc.record_step()
    assert "forward_ms" in mc.get_average()
    f = F.create_fsdp2_from_dict({"fsdp_sharding_strategy": "shard_grad_op", "fsdp_mixed_precision": "fp32",
                                  "gradient_checkpointing": False, "max_grad_norm": 0.5, "unknown_key": 1})
    assert f.config.gradient_clipping_norm == 0.5 and not f.config.activation_checkpointing
    assert F.detect_hardware().is_err() or F.detect_hardware().unwrap().sm_count > 0


def _chain(n=8):
    torch.manual_seed(0)
    return nn.Sequential(*[nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(n)])


@pytest.mark.parametrize("sched,P,V,M,ckpt", [("gpipe", 4, 1, 4, False), ("1f1b", 4, 1, 8, True),
                                              ("interleaved", 2, 2, 4, False), ("zero_bubble", 4, 1, 8, False),
                                              ("chimera", 4, 1, 8, False)])
def test_pipeline_schedules_in_one_process(sched, P, V, M, ckpt):
    from trainscale_b200.parallel import pipeline as PL
    x, y = torch.randn(16, 16), torch.randn(16, 16)
    ref = _chain()
    loss_ref = nn.functional.mse_loss(ref(x), y)
    loss_ref.backward()
    m = _chain()
    cfg = PL.PipelineConfig(num_stages=P, num_virtual_stages=V, num_microbatches=M, schedule=sched,
                            memory=PL.MemoryConfig(enable_activation_checkpointing=ckpt))
    stages = PL.split_model_into_stages(m, P if sched == "chimera" else P * V, checkpoint_activations=ckpt)
    pipe = PL.PipelineParallel(stages, cfg, nn.functional.mse_loss)
    with PL.pipeline_profiler(pipe, sched) as rep:
        loss = pipe(PL.split_into_microbatches(x, M), PL.split_into_microbatches(y, M))
    assert abs(float(loss) - float(loss_ref)) < 1e-6
    for a, b in zip(m.parameters(), ref.parameters()):
        torch.testing.assert_close(a.grad, b.grad, rtol=1e-5, atol=1e-7)
    assert rep["forwards"] == rep["backwards"] == M * len(stages) * (1 if sched != "chimera" else 1)
    assert (rep["weight_grads"] > 0) == (sched == "zero_bubble")


def test_chimera_order_and_balancing():
    from trainscale_b200.parallel import pipeline as PL
    acts = PL.chimera_schedule(4, 8)
    for w, lst in enumerate(acts):
        assert sum(a.op == "F" for a in lst) == 8 and sum(a.op == "B" for a in lst) == 8
        assert {a.mb for a in lst if a.chunk == 0} == {0, 1, 2, 3} and {a.mb for a in lst if a.chunk == 1} == {4, 5, 6, 7}
    # both ends start a forward at once: the fill bubble of a one-directional pipeline is halved
    assert acts[0][0] == PL.Action("F", 0, 0) and acts[3][0] == PL.Action("F", 4, 1)
    with pytest.raises(ValueError):
        PL.chimera_schedule(3, 8)
    layers = [nn.Linear(64, 64) for _ in range(6)] + [nn.Linear(64, 4096), nn.Linear(4096, 64)]
    r = PL.balance_stages_by_memory(layers, 4)
    assert sum(len(x) for x in r) == 8 and len(r) == 4
    heavy = max(range(4), key=lambda s: sum(PL.estimate_stage_memory(layers[i])["total"] for i in r[s]))
    assert len(r[heavy]) <= 2                      # the two large layers do not share a stage with many others
    assert float(PL.merge_microbatches([torch.tensor(1.0), torch.tensor(3.0)])) == 2.0
    pool = PL.TensorPool()
    t = pool.allocate((4, 4))
    pool.deallocate(t)
    assert pool.allocate((4, 4)).data_ptr() == t.data_ptr() and pool.stats()["reuses"] == 1


def test_pipeline_api_across_ranks():
    r = launch("pipeline_api.py", 2, 29682)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT ok=True" in r.stdout


def test_zbpp_schedule_optimizer_and_partitioner():
    import itertools
    from trainscale_b200.parallel import pp as PP
    from trainscale_b200.parallel import zbpp as Z
    prof = [Z.StageProfile(100, 100, 100, 1 << 20, 1 << 22, 0, 0) for _ in range(4)]
    base = PP.simulate([PP.one_f_one_b_schedule(s, 4, 8) for s in range(4)])["bubble_fraction"]
    h1 = Z.ZBPPScheduleOptimizer(Z.ScheduleConfig(4, 8, 1 << 30, prof)).optimize()
    h2 = Z.ZBPPScheduleOptimizer(Z.ScheduleConfig(4, 8, 1 << 30, prof, enable_interleaving=False)).optimize()
    assert h2.bubble_fraction < h1.bubble_fraction < base
    assert max(h1.peak_memory_bytes.values()) <= (1 << 22) + 4 * (1 << 20)         # ZB-H1: no more than 1F1B's stage 0
    tight = Z.ZBPPScheduleOptimizer(Z.ScheduleConfig(4, 8, (1 << 22) + 2 * (1 << 20), prof)).optimize()
    assert max(tight.peak_memory_bytes.values()) <= (1 << 22) + 2 * (1 << 20)
    with pytest.raises(ValueError):
        Z.ZBPPScheduleOptimizer(Z.ScheduleConfig(4, 8, 1 << 22, prof)).optimize()
    for st, lst in h1.schedule.items():                                            # every op once, W after its B
        for op in (Z.OpType.FORWARD, Z.OpType.BACKWARD_INPUT, Z.OpType.BACKWARD_PARAMS):
            assert sorted(s.microbatch_id for s in lst if s.op_type == op) == list(range(8))
        pos = {(s.op_type, s.microbatch_id): i for i, s in enumerate(lst)}
        assert all(pos[(Z.OpType.BACKWARD_PARAMS, m)] > pos[(Z.OpType.BACKWARD_INPUT, m)] for m in range(8))
    costs = [3, 1, 4, 1, 5, 9, 2, 6]
    b = Z.ModelPartitioner._dp_partition(costs, 3)
    got = max(sum(costs[b[j]:b[j + 1]]) for j in range(3))
    brute = min(max(sum(costs[:i]), sum(costs[i:j]), sum(costs[j:])) for i, j in itertools.combinations(range(1, 8), 2))
    assert got == brute


def test_zbpp_pipeline_with_sync_bypass_matches_global_clip():
    import copy
    from trainscale_b200.optim import AdamW
    from trainscale_b200.parallel import zbpp as Z
    torch.manual_seed(0)
    model = nn.Sequential(*[nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(8)])
    ref = copy.deepcopy(model)
    x, y = torch.randn(16, 16), torch.randn(16, 16)
    # a threshold far below the gradient norm: every optimistic local step must be rolled back and redone
    pipe = Z.create_zbpp_pipeline(model, 4, 8, lr=1e-2, weight_decay=0.0, max_grad_norm=0.05)
    opt = AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    for _ in range(3):
        loss = pipe.train_step(x, y)
        lr_ = nn.functional.mse_loss(ref(x), y)
        lr_.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05)
        opt.step()
        opt.zero_grad()
        assert abs(float(loss) - float(lr_)) < 1e-5
    assert pipe.finalize() == 4
    assert all(o.rollbacks >= 1 for o in pipe.engine.optimizers)
    for a, b in zip(pipe.parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    rep = Z.ZBPPBenchmark(pipe, x, y).run_all()
    assert rep["passed"] and rep["schedule"]["bubble_fraction"] < rep["schedule"]["one_f_one_b_bubble"]
    st = Z.PipelineStageModule(nn.Linear(4, 4))
    inp = torch.randn(2, 4)                       # no input gradient needed: the weight work must still be parked
    st(inp).sum().backward()
    assert st.module.weight.grad is None and st.num_deferred == 1
    st.execute_deferred_b_params()
    torch.testing.assert_close(st.module.weight.grad, inp.sum(0).expand(4, 4))


def test_grad_buffer_zero1_two_ranks():
    r = launch("grad_buffer_zero1.py", 2, 29684)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT ok=True" in r.stdout


def test_dist_kernels_four_ranks():
    r = launch("dist_kernels_case.py", 4, 29686)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT ok=True" in r.stdout


def test_gradient_compressor_and_buckets():
    from trainscale_b200.parallel import dist_kernels as DK
    torch.manual_seed(0)
    g = torch.randn(64, 32)
    c = DK.GradientCompressor(topk_ratio=0.1)
    payload, ctx = c.compress(g, key="w")
    out = c.decompress(payload, ctx)
    assert int((out != 0).sum()) == int(64 * 32 * 0.1)
    torch.testing.assert_close(out + c._error_buffers["w"], g)              # nothing is lost, only delayed
    payload2, ctx2 = c.compress(torch.zeros_like(g), key="w")               # the residual comes back next step
    assert float(c.decompress(payload2, ctx2).abs().sum()) > 0
    low = torch.randn(64, 4) @ torch.randn(4, 32)
    p = DK.GradientCompressor(use_powersgd=True, powersgd_rank=4)
    for _ in range(3):                                                       # power iteration converges on rank 4
        payload, ctx = p.compress(low, key="m")
        p._error_buffers.pop("m")
    torch.testing.assert_close(p.decompress(payload, ctx), low, rtol=1e-3, atol=1e-3)
    assert sum(t.numel() for t in payload) < low.numel() / 4
    cast, ctx = DK.GradientCompressor(use_bf16=True).compress(g)
    assert cast[0].dtype is torch.bfloat16 and DK.GradientCompressor().decompress(cast, ctx).dtype is torch.float32
    ts = [torch.zeros(100), torch.zeros(100), torch.zeros(10, dtype=torch.float64), torch.zeros(300)]
    buckets = DK.BucketManager(bucket_size_mb=1000 / 2 ** 20).create_buckets(ts)
    assert [len(b.tensors) for b in buckets] == [2, 1, 1]
    k = DK.DistributedKernels()                                              # no process group: identities
    x = torch.ones(3)
    assert k.all_reduce(x) is x and k.all_gather(x) is x and k.reduce_scatter(x) is x
    assert DK.get_world_info()[1] == 1 and DK.get_distributed_backend() is DK.DistributedBackend.NONE
    z = DK.ZeroCopyTransfer("cpu")
    assert z.host_to_device(x) is x and z.device_to_host(x) is x


def test_tensor_parallel_blocks_two_ranks():
    r = launch("tp_blocks.py", 2, 29688)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT ok=True" in r.stdout and r.stdout.count("ok=True") >= 3


def test_context_parallel_engine_two_ranks():
    r = launch("cp_engine.py", 2, 29690)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT ok=True" in r.stdout


def test_context_parallel_helpers():
    from trainscale_b200.parallel import cp as CP
    a = CP.TensorArena(4096)
    t = a.allocate((10, 10), torch.float32)
    assert t.is_ok() and t.unwrap().shape == (10, 10) and a.allocate((1000,), torch.float32).is_err()
    a.reset()
    assert a.available_bytes == 4096
    pool = CP.RingBufferPool(2, (4,), torch.float32)
    _, i = pool.get_compute_buffer()
    _, j = pool.get_recv_buffer()
    with pytest.raises(RuntimeError):
        pool.get_compute_buffer()
    pool.mark_free(i)
    assert pool.get_compute_buffer()[1] == i and j != i
    s = CP.BalancedCPScheduler(CP.HybridCPConfig(8192, 8))
    L = [30000, 9000, 4000, 4000, 2000, 1000, 500, 500, 400]
    plan = s.balanced_schedule(L)
    assert all(plan[g] for g in range(8))                                     # nobody idles
    assert sorted({i for g in plan for i, _ in g}) == list(range(len(L)))
    assert [cp for i, cp in plan[0] if i == 0] == [4] and s.get_total_workload(30000) == 30000 ** 2 / 4
    grp, nxt = s.next_hdp_group(L)
    assert sum(cp for _, cp in grp) <= 8 and nxt == len(grp)
    assert CP.create_context_parallel_engine(2).is_err() and CP.create_context_parallel_engine(1, "bogus").is_err()
    assert CP.ContextParallelConfig.from_dict({"cp_degree": 1, "load_balancer": "zigzag", "junk": 1}).is_ok()
    seen = []
    CP.hybrid_context_parallel_forward_backward(lambda b, cp, slot: seen.append((b["input_ids"].shape[1], cp, slot)),
                                                [{"input_ids": torch.zeros(1, n)} for n in L], s, rank=1)
    assert seen[0] == (30000, 4, 1)


def test_utility_surface_single_process():
    import copy
    import tempfile
    from trainscale_b200.parallel import activation as A
    from trainscale_b200.parallel import ddp as DDP
    from trainscale_b200.parallel import dist_utils as U
    from trainscale_b200.parallel import mesh as M
    from trainscale_b200.utils.cuda_graphs import InductorConfigManager
    # memory pressure monitor on a fake probe
    used = [10]
    mon = DDP.MemoryPressureMonitor(probe=lambda: (used[0], 100))
    assert mon.check() == "normal" and mon.suggested_bucket_mb(80) == 80
    used[0] = 90
    assert mon.check() == "high" and mon.suggested_bucket_mb(80) == 40
    used[0] = 97
    assert mon.check() == "critical" and mon.suggested_bucket_mb(80) == 20 and len(mon.events) == 2
    t = DDP.CUDATimer("cpu")
    with t:
        pass
    assert t.elapsed_ms() >= 0 and DDP.SyncMode("local_sgd") is DDP.SyncMode.LOCAL_SGD
    assert DDP.DDPMetrics(allreduce_ms=1.0, bytes_reduced=10 ** 9).bus_bandwidth_gbs(8) == pytest.approx(1750.0)
    # hierarchical recomputation == plain backward
    torch.manual_seed(0)
    layers = nn.ModuleList([nn.Sequential(nn.Linear(8, 8), nn.Tanh()) for _ in range(9)])
    ref = copy.deepcopy(layers)
    x = torch.randn(4, 8, requires_grad=True)
    x2 = x.detach().clone().requires_grad_(True)
    h = A.HierarchicalCheckpointManager(layers)
    h(x).sum().backward()
    z = x2
    for l in ref:
        z = l(z)
    z.sum().backward()
    assert h.group_size == 3 and h.kept_tensors() == 6
    torch.testing.assert_close(x.grad, x2.grad)
    for a, b in zip(layers.parameters(), ref.parameters()):
        torch.testing.assert_close(a.grad, b.grad)
    assert A.CheckpointFunction.__name__ == "CheckpointFunction"
    pool = A.ActivationPool()
    buf = pool.get((4, 4), torch.float32, "cpu")
    pool.put(buf)
    assert pool.get((4, 4), torch.float32, "cpu").data_ptr() == buf.data_ptr() and pool.hits == 1
    # mesh views
    cfg = M.ParallelDimsConfig(dp_replicate=2, dp_shard=-1, cp=2, tp=2, pp=2, world_size=32)
    v = M.MeshCache.views(cfg, rank=13)
    assert v["dense"].size("fsdp") == 4 and v["loss"].size() == 8 and v["dataloading"].shape == (2, 4, 2, 2)
    assert M.MeshCache.get(cfg, rank=13) is M.MeshCache.get(cfg, rank=13)
    with pytest.raises(KeyError):
        v["loss"].get_group("tp")
    # engine factory + checkpoint helpers
    from trainscale_b200.models.llama import LlamaConfig, build_model
    m = build_model(LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                num_attention_heads=2, num_key_value_heads=2, head_dim=16), dtype=torch.float32,
                    device="cpu", seed=0)
    m, eng = U.prepare_model_for_distributed(m, "zero2", device="cpu", param_dtype=torch.float32, lr=1e-2)
    ids = torch.randint(0, 64, (2, 8))
    eng.backward(m(ids, labels=ids).loss)
    eng.step()
    d = tempfile.mkdtemp()
    U.save_checkpoint_distributed(d, m, eng, {"step": 1})
    w = {k: t.clone() for k, t in m.state_dict().items()}
    with torch.no_grad():
        for p in m.parameters():
            p.zero_()
    assert U.load_checkpoint_distributed(d, m, eng) == {"step": 1}
    assert all(torch.equal(w[k], t) for k, t in m.state_dict().items())
    with pytest.raises(ValueError):
        U.prepare_model_for_distributed(m, "bogus", device="cpu")
    assert U.DeviceManager().device.type in ("cpu", "cuda") and U.HardwareTopology.detect().num_gpus >= 0
    assert U.get_process_group("world") is None
    # inductor options only touch torch when asked to, and are restored
    import torch._inductor.config as ic
    before = ic.max_autotune
    with InductorConfigManager(apply_to_torch=True).for_mode("max-autotune") as mgr:
        assert ic.max_autotune is True and mgr.compilation_config().mode == "cuda_graphs"
    assert ic.max_autotune == before and InductorConfigManager(max_autotune=True).apply() == {}


def test_registry_module_patchers_keep_the_maths():
    transformers = pytest.importorskip("transformers")
    from trainscale_b200.registry import auto_patch, auto_patch_layernorm
    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2)
    torch.manual_seed(0)
    m = transformers.LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 128, (1, 16))
    with torch.no_grad():
        ref = m(ids).logits
    counts = auto_patch(m)
    assert counts["layernorm"] == 5 and counts["mlp"] == 2 and counts["fp8_linear"] == 0
    with torch.no_grad():
        torch.testing.assert_close(m(ids).logits, ref)
    assert auto_patch(m)["layernorm"] == 0                       # idempotent
    ln = nn.Sequential(nn.LayerNorm(16))
    x = torch.randn(2, 16)
    want = ln(x)
    assert auto_patch_layernorm(ln) == 1
    torch.testing.assert_close(ln(x), want)


def test_expert_parallel_decoder_two_ranks():
    r = launch("ep_decoder.py", 2, 29697)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == 2


@pytest.mark.parametrize("nproc,port", [(2, 29703), (4, 29704)])
def test_ulysses_attention_matches_full_attention(nproc, port):
    r = launch("ulysses.py", nproc, port)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT ok=True" in r.stdout


def test_activation_checkpoint_reference_surface():
    import torch
    import torch.nn as nn

    from trainscale_b200.models.llama import LlamaConfig, build_model
    from trainscale_b200.parallel import activation as A
    # the decoder obeys no_checkpoint / force_checkpoint
    m = build_model(LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                num_attention_heads=2, num_key_value_heads=2, head_dim=16), dtype=torch.float32,
                    device="cpu", seed=0)
    m.gradient_checkpointing_enable(1)
    ids = torch.randint(0, 64, (1, 8))
    calls = []
    import trainscale_b200.models.llama as L
    real = L.checkpoint
    L.checkpoint = lambda fn, *a, **k: (calls.append(1), real(fn, *a, **k))[1]
    try:
        m.train()
        base = m(ids, labels=ids).loss
        assert len(calls) == 2
        with A.no_checkpoint():
            assert torch.allclose(m(ids, labels=ids).loss, base) and len(calls) == 2
        m.eval()
        m(ids, labels=ids)
        assert len(calls) == 2
        with A.force_checkpoint():
            m(ids, labels=ids)
        assert len(calls) == 4
    finally:
        L.checkpoint = real
    # functional checkpoint with keyword arguments, segments, operation contexts
    lin = nn.Linear(4, 4)
    x = torch.randn(3, 4, requires_grad=True)
    y = A.checkpoint(lambda t, scale=1.0: lin(t) * scale, x, scale=2.0)
    y.sum().backward()
    assert torch.allclose(y, lin(x) * 2) and x.grad is not None
    layers = nn.ModuleList(nn.Linear(4, 4) for _ in range(6))
    seg = A.CheckpointSegment(0, 0, 6, level=1)
    kids = seg.split(4)
    assert [len(k) for k in kids] == [1, 2, 1, 2] and 3 in kids[2] and kids[0].level == 0
    want = x
    for l_ in layers:
        want = l_(want)
    assert torch.allclose(seg.run(layers, x), want, atol=1e-6)
    with A.OperationCheckpointContext(None, "layernorm") as ctx:
        assert A.OperationCheckpointContext.active() == ["layernorm"] and ctx.should_checkpoint()
        assert torch.allclose(ctx.run(torch.nn.functional.layer_norm, x, (4,)), torch.nn.functional.layer_norm(x, (4,)))
        with A.no_checkpoint():
            assert torch.allclose(ctx.run(lin, x), lin(x))
    assert not A.OperationCheckpointContext(None, "attention").should_checkpoint()
    # records
    h = A.OffloadHandle.offload(7, x.detach(), A.OffloadTarget.CPU_PAGED)
    assert torch.equal(h.restore(), x.detach()) and h.shape == (3, 4)
    import pytest
    with pytest.raises(ValueError):
        A.OffloadHandle(1, (1,), torch.float32, torch.device("cpu"), A.OffloadTarget.NVME)
    snap = A.MemorySnapshot.take()
    assert snap.timestamp_ns > 0 and A.CheckpointImpl.NO_REENTRANT.value == "no_reentrant"
    assert A.LayerProfile("l0", A.OperationType.FFN, 1, 2, 0.5, False, True).is_ffn
    assert A.CheckpointMetrics("l0", 1, 2, 3, 4, 5).memory_saved_bytes == 3
    ac = A.create_activation_checkpoint("selective", frequency=3)
    assert ac.cfg.frequency == 3 and A.create_activation_checkpoint("op_selective").cfg.mode == A.CheckpointMode.OP_SELECTIVE


def test_mesh_topology_records_and_tensor_parallel_helpers():
    import torch

    from trainscale_b200.parallel import mesh as M
    from trainscale_b200.parallel import tp as T
    r = M.create_parallel_dims(16, tp=2, pp=2, cp=2, rank=5)
    assert r.is_ok() and r.unwrap().sizes == {"pp": 2, "dp_replicate": 1, "dp_shard": 2, "cp": 2, "tp": 2}
    assert M.create_parallel_dims(6, tp=4).is_err()
    specs = {d.name: d for d in M.DimensionSpec.of(M.ParallelDimsConfig(tp=2, world_size=8))}
    assert specs["dp_shard"].degree == 4 and specs["tp"].is_sharding and not specs["pp"].requires_comm
    import pytest
    with pytest.raises(ValueError):
        M.DimensionSpec("bogus", 2, M.ParallelDimType.DATA)
    topo = M.detect_cluster_topology()
    assert topo.num_nodes >= 1 and topo.nodes[0].num_gpus == topo.gpus_per_node
    assert M.GPUArchitecture.from_compute_capability((10, 0)) is M.GPUArchitecture.BLACKWELL
    assert M.GPUArchitecture.from_compute_capability((9, 0)) is M.GPUArchitecture.HOPPER
    assert M.InterconnectType.NVLINK5 == 4 and M.CommunicationAlgorithm.RING == 1 and M.HardwareVendor.NVIDIA == 1
    assert M.ParallelDimsMetrics(num_cache_hits=3, num_cache_misses=1).to_dict()["cache_hit_rate"] == 0.75

    with T.tensor_parallel_context(T.TensorParallelConfig()) as mgr:
        assert mgr.initialized and T.get_tensor_parallel_world_size() == 1 and T.get_sequence_parallel_rank() == 0
        assert not T.is_sequence_parallel_enabled() and T.get_tensor_parallel_group() is None
        net = torch.nn.Sequential(T.FusedColumnParallelLinearWithGELU(8, 16),
                                  T.FusedRowParallelLinearWithDropout(16, 8, dropout_prob=0.1), torch.nn.LayerNorm(8)).eval()
        x = torch.randn(3, 8)
        F = torch.nn.functional
        want = F.linear(F.gelu(F.linear(x, net[0].linear.weight, net[0].linear.bias), approximate="tanh"),
                        net[1].linear.weight, net[1].linear.bias)
        assert torch.allclose(net[1](net[0](x)), want, atol=1e-5)
        counts = T.compute_parameter_count(net)
        assert counts["parallel_params"] == 280 and counts["replicated_params"] == 16 and counts["total_params"] == 296
    with pytest.raises(ValueError):
        T.TensorParallelConfig(tensor_parallel_size=3)
    assert T.CommStats(1, 2, 3, "all_reduce").latency_ns == 3


def test_dist_utils_expert_parallel_and_ddp_reference_names(tmp_path):
    import pytest
    import torch

    from trainscale_b200.parallel import ddp as D
    from trainscale_b200.parallel import dist_utils as U
    from trainscale_b200.parallel import ep as E
    T_ = U.DistributedStateTransition
    assert T_.allowed(U.StatePhase.INITIALIZING, U.StatePhase.READY) and T_.allowed(U.StatePhase.READY, U.StatePhase.ERROR)
    assert not T_.allowed(U.StatePhase.READY, U.StatePhase.INITIALIZING)
    assert U.GradientConfig().max_norm == 1.0 and U.DistributedStrategy.FSDP2.value == "fsdp2"
    t = torch.ones(2)
    assert U.dist_scatter(t) is t and U.prepare_scheduler_for_distributed("s") == "s"
    opt = torch.optim.SGD([torch.nn.Parameter(t)], lr=0.1)
    assert U.prepare_optimizer_for_distributed(opt, None) is opt
    with pytest.raises(ValueError):
        U.prepare_optimizer_for_distributed(opt, None, U.DistributedStrategy.FSDP2)
    with U.mixed_precision_context(dtype=torch.bfloat16):
        assert torch.nn.functional.linear(torch.randn(2, 4), torch.randn(3, 4)).dtype == torch.bfloat16
    U.print_rank_0("rank 0 prints")

    cfg = E.ExpertParallelConfig(num_experts=4, top_k=2, hidden_size=16, capacity_factor=1.0, min_capacity=1)
    out = E.RouterBase(cfg)(torch.randn(2, 6, 16))
    T, C = 12, out.metadata["capacity"]
    assert out.dispatch_mask.shape == (T, 4, C) and out.expert_indices.shape == (T, 2)
    assert int(out.dispatch_mask.sum()) + out.metadata["dropped"] == T * 2
    assert out.dispatch_mask.sum(0).max() <= 1                      # one token per (expert, slot)
    kept = out.dispatch_mask.any(-1)
    assert torch.allclose(out.combine_weights.sum(-1)[kept], torch.zeros(T, 4).scatter(1, out.expert_indices, out.expert_weights)[kept])
    probs = torch.softmax(out.router_logits, -1)
    sw = E.load_balance_loss(E.LoadBalanceLossType.SWITCH, probs, out.expert_indices)
    st = E.load_balance_loss(E.LoadBalanceLossType.STMOE, probs, out.expert_indices, out.router_logits)
    assert float(st) > float(sw) > 0 and float(E.load_balance_loss(E.LoadBalanceLossType.VMOE, probs, out.expert_indices)) >= 0
    assert E.get_expert_parallel_rank() == 0 and E.get_expert_parallel_world_size() == 1
    assert E.RoutingStrategy.EXPERT_CHOICE.value == "expert_choice"

    class Half(D.GradientCompressionHook):
        def compress(self, bucket):
            return bucket.half()
    b = torch.tensor([1.0, 2.0, 3.0])
    assert torch.equal(Half()(None, b), torch.tensor([1.0, 2.0, 3.0]))
    assert D.BucketSchedule.REVERSE == 1 and D.AllReduceAlgorithm.NCCL_AUTO == 3
    y = tmp_path / "ddp.yaml"
    y.write_text("distributed:\n  ddp:\n    bucket_cap_mb: 64\n    gradient_compression: bf16\n")
    r = D.create_ddp_from_yaml(str(y))
    assert r.is_ok() and r.unwrap().config.bucket_cap_mb == 64
    assert D.create_ddp_from_yaml(str(tmp_path / "missing.yaml")).is_err()


def test_parallel_dims_state_pool_timer_and_manager_accessors():
    import torch

    from trainscale_b200.parallel import dist_utils as U
    from trainscale_b200.parallel import mesh as M
    from trainscale_b200.parallel import tp as T
    d = M.ParallelDims.create(16, tp=2, cp=2, pp=2, rank=3).unwrap()
    assert d.tp_enabled and d.cp_enabled and d.pp_enabled and d.dp_shard_enabled and not d.ep_enabled
    assert d.fsdp_gradient_divide_factor == 4 and d.non_data_parallel_size == 8 and d.seq_len_divisor == 8
    assert d.config.tp == 2 and d.device_type in ("cpu", "cuda")
    views = d.build_mesh().unwrap()
    assert views["dense"].shape == (2, 1, 4, 2) and d.build_mesh().unwrap() is views
    assert d.get_mesh(["dp_shard", "tp"]).shape == (2, 2) and d.get_optional_mesh("ep") is None
    assert sorted(d.get_all_1d_meshes()) == ["cp", "dp_shard", "pp", "tp"] and d.world_mesh.size() == 16
    import pytest
    with pytest.raises(ValueError):
        d.get_mesh("dp_replicate")
    with pytest.raises(ValueError):
        d.get_optional_mesh("bogus")
    d.get_mesh("tp")
    d.get_mesh("tp")
    assert d.metrics.num_cache_hits >= 1 and d.metrics.compute_cache_hit_rate() > 0
    assert isinstance(d.get_communication_algorithm(1 << 20), M.CommunicationAlgorithm)
    assert d.estimate_memory_per_gpu(8_000_000_000, 16, 8192, 4096, 32) > 2 ** 30
    assert isinstance(M.HardwareDetector.detect_architecture(), M.GPUArchitecture)
    assert M.HardwareDetector.get_optimal_device_order() == list(range(M.HardwareDetector.detect()["num_gpus"]))
    M.MeshCache.set_global("dense", d.world_mesh)
    assert M.MeshCache.get_global("dense") is not None and M.MeshCache.get_world() is None
    M.MeshCache.clear()

    st = U.DistributedState.from_environment()
    assert st.is_main_process and st.is_local_main and not st.is_distributed and st.is_initialized and st.num_nodes == 1
    t = torch.ones(3)
    assert st.all_reduce(t, "mean") is t and st.broadcast(t) is t and st.get_data_parallel_group() is None
    pool = st.tensor_pool
    a = pool.acquire((3, 5))
    pool.release(a)
    b = pool.acquire(15)
    assert a.data_ptr() == b.data_ptr() and pool.get_stats()["hit_rate"] == 0.5
    pool.free()
    assert pool.get_stats()["pooled_bytes"] == 0
    tm = U.NanoTimer().start()
    sum(range(10000))
    assert tm.stop().elapsed_ns() > 0 and abs(tm.elapsed_ms() * 1e3 - tm.elapsed_us()) < 1e-6
    with U.CUDATimer() as t2:
        pass
    assert t2.sync_and_elapsed_ms() >= 0
    m = torch.nn.Linear(2, 2)
    m(torch.ones(1, 2)).sum().backward()
    g0 = m.weight.grad.clone()
    gs = U.GradScaler(init_scale=4.0, growth_interval=1)
    assert gs.unscale_(parameters=m.parameters()) and torch.allclose(m.weight.grad, g0 / 4)
    gs.update()
    assert gs.get_scale() == 8.0
    m.weight.grad[0, 0] = float("inf")
    assert not gs.unscale_(parameters=m.parameters())
    gs.update()
    assert gs.get_scale() == 4.0
    assert U.DistributedManager.get_instance() is U.DistributedManager()
    assert U.DeviceManager.auto_detect().compute_capability >= (0, 0)
    mgr = T.ProcessGroupManager.get_instance().initialize(1, 1)
    assert mgr.is_initialized() and mgr.get_world_size("tensor") == 1 and mgr.get_rank("data") == 0
    assert mgr.get_group("sequence") is None
    buf = mgr.acquire_buffer((4, 4))
    mgr.release_buffer(buf)
    mgr.destroy()


# ------------------------------------------------------------------------------------------------ offload protocol, policy members
def test_pipeline_offload_manager_schedule_protocol():
    """Chunks are offloaded in forward and brought back in backward with gradients equal to the plain run; the
    backward order is learnt in the first iteration and replayed; disabling offload keeps everything in place."""
    import torch
    from trainscale_b200.parallel.activation import PipelineOffloadManager
    PipelineOffloadManager.reset_instance()
    m = PipelineOffloadManager.get_instance()
    assert m is PipelineOffloadManager.get_instance()
    lin = torch.nn.Linear(64, 64)

    def iteration():
        outs, grads = [], []
        for _ in range(3):
            m.init_model_chunk_offload_handler(min_offload_tensor_size=128)
            m.cur_forward_chunk().begin_group("mlp")
            x = torch.randn(8, 64, requires_grad=True)
            with m:
                outs.append((x, (lin(x).relu() ** 2).sum()))
        for x, y in outs:
            m.pop_backward_chunk("mlp")
            y.backward()
            if m.cur_backward_chunk() is not None:
                assert m.cur_backward_chunk().finish_all_groups("mlp")
            grads.append(x.grad.clone())
        return outs, grads

    outs, grads = iteration()
    first = m.offload_summary_total_bytes
    assert first > 0 and m.offload_summary_bytes == {"mlp": first}
    x = outs[0][0].detach().clone().requires_grad_(True)
    (lin(x).relu() ** 2).sum().backward()
    assert torch.allclose(x.grad, grads[0])
    m.reset()
    iteration()
    assert len(m._forward) == 3 and m.offload_summary_total_bytes == 2 * first     # same three chunks, replayed
    m.disable_offload()
    m.reset()
    iteration()
    assert m.offload_summary_total_bytes == 2 * first
    m.enable_offload()
    assert m.cpu_tensor_pool is m.cur_forward_chunk().cpu_tensor_pool
    # interleaved (virtual) stages: within one round the later virtual stage goes to backward first
    PipelineOffloadManager.reset_instance()
    m = PipelineOffloadManager.get_instance()
    for _ in range(2):
        for stage in range(2):
            m.init_model_chunk_offload_handler(2, stage)
    m._flush(final=True)
    assert [(h.vpp_rank, h.chunk_id) for h in m._backward] == [(1, 1), (0, 0), (1, 3), (0, 2)]
    PipelineOffloadManager.reset_instance()


def test_chunk_handler_tags_and_group_bookkeeping():
    import pytest
    import torch
    from trainscale_b200.parallel.activation import ChunkOffloadHandler, OffloadTensorGroup
    h = ChunkOffloadHandler(min_offload_tensor_size=16)
    assert h.is_empty_chunk() and h.finish_all_groups()
    h.begin_group("attn")
    small, big = torch.ones(4), torch.arange(64.0)
    s1, s2 = h.tensor_push(small), h.tensor_push(big)
    assert s1[0] == "direct" and s2[0] == "offloaded" and not h.is_empty_chunk("attn") and h.is_empty_chunk("mlp")
    assert not h.finish_all_groups("attn")
    assert h.tensor_pop(s1) is small and torch.equal(h.tensor_pop(s2), big)
    assert h.finish_all_groups("attn") and h.get_max_deduplicated_groups() == 1
    with pytest.raises(ValueError):
        h.tensor_pop(("bogus", None))
    h.reset()
    assert h.is_empty_chunk()
    g = OffloadTensorGroup("g")
    g.push_tensor("k", small)
    g.update_stats(small)
    assert g.pop_tensor("k") is small and g.total_offload_bytes == 16 and g.total_tensor_count == 1


def test_activation_policy_members():
    import torch
    import torch.nn as nn
    from trainscale_b200.models.llama import build_model
    from trainscale_b200.parallel.activation import (ActivationCheckpoint, ActivationCheckpointConfig, ActivationOffloader,
                                                     ActivationPool, CheckpointMetrics, HierarchicalCheckpointManager,
                                                     LayerProfile, MemoryProfiler, OperationCheckpointContext,
                                                     OperationType, SelectiveCheckpointPolicy)
    mp = MemoryProfiler()
    mp.clear()
    flash = mp.estimate_activation_memory(1, 4096, 4096, 32, 32, 14336, torch.bfloat16, 8)
    dense = mp.estimate_activation_memory(1, 4096, 4096, 32, 32, 14336, torch.bfloat16, 8, flash_attention=False)
    # per token and layer: 5 H + (nh + 2 nkv) d + 3 I elements
    per_token = (5 * 4096 + 48 * 128 + 3 * 14336) * 2
    assert flash == int((4096 * per_token + 32 * 4096 * 4) * 32 * 1.1)
    assert abs((dense - flash) - 32 * 4096 * (4096 * 2 - 4) * 32 * 1.1) <= 2      # the S x S probabilities

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(16, 64), nn.Linear(64, 16)
        def forward(self, x):
            return self.b(torch.relu(self.a(x)))

    prof = mp.profile_layer(MLP(), "mlp0", torch.randn(2, 8, 16))
    assert prof.operation_type is OperationType.FFN and prof.is_ffn
    assert prof.activation_memory_bytes == (2 * 8 * 16 + 2 * 8 * 64) * 4          # the input and the ReLU output
    mp.record_checkpoint_metrics(CheckpointMetrics("l", 1, 2, 100, 1, 1))
    st = mp.get_statistics()
    assert st["profiled_layers"] == 1 and st["total_memory_saved_bytes"] == 100 and st["total_recompute_time_ns"] == 2
    mp.clear()
    assert mp.get_statistics()["checkpoint_operations"] == 0

    pol = SelectiveCheckpointPolicy()
    assert pol.should_checkpoint("self_attn") and not pol.should_checkpoint("input_layernorm")
    assert not pol.should_checkpoint("mlp", recompute_cost=0.01)                  # switched on, but trivially cheap
    assert pol.should_checkpoint("other", activation_size_bytes=10 ** 9)
    assert pol.should_checkpoint("other", 10, 0.5, memory_pressure=0.9)
    assert not pol.should_checkpoint("other", 10, 0.5, memory_pressure=0.1)
    pol.update_from_profile(LayerProfile("other", OperationType.CUSTOM, 10 ** 9, 0, 0.5, False, False))
    assert pol.should_checkpoint("other", 10, 0.5, memory_pressure=0.1)

    h = HierarchicalCheckpointManager(ActivationCheckpointConfig(segment_size=4, hierarchy_levels=3), 20)
    assert [(s.start_layer, s.end_layer) for s in h._level(1)] == [(0, 8), (8, 16), (16, 20)]
    assert h.should_checkpoint_layer(3) and not h.should_checkpoint_layer(4)
    assert h.adjust_level_for_memory(0.5) == 2 and h.should_checkpoint_layer(15) and not h.should_checkpoint_layer(7)
    assert h.adjust_level_for_memory(0.9) == 1 and h.adjust_level_for_memory(0.99) == 0
    assert h.get_segment_for_layer(19, level=0).start_layer == 16

    pool = ActivationPool()
    t = pool.acquire((4, 4), torch.float32)
    pool.release(t)
    assert pool.acquire((4, 4), torch.float32) is not None and pool.hit_rate == 0.5 and pool.get_stats()["hits"] == 1

    off = ActivationOffloader()
    x = torch.randn(8, 8)
    hid = off.offload(x)
    off.prefetch(hid)
    assert torch.equal(off.reload(hid), x)
    off.release(hid)
    off.clear()

    m = build_model("tiny", dtype=torch.float32, device="cpu")
    L = len(m.model.layers)
    assert ActivationCheckpoint.apply_full(m)._ts_checkpointed_layers == list(range(L))
    assert ActivationCheckpoint.apply_selective(m, 2)._ts_checkpointed_layers == list(range(0, L, 2))
    assert ActivationCheckpoint.apply_hierarchical(m, 2, 2)._ts_checkpointed_layers == [i for i in range(L) if i % 2 == 0]
    assert ActivationCheckpoint.apply_memory_budget(m, 0.7, 1, 128, total_bytes=1 << 24)._ts_checkpointed_layers == list(range(L))
    huge = ActivationCheckpoint.apply_memory_budget(m, 0.7, 1, 128, total_bytes=1 << 40)
    assert huge._ts_checkpointed_layers == [] and huge._ts_activation_checkpoint.get_statistics()["config"]["mode"] == "MEMORY_BUDGET"

    with OperationCheckpointContext(pol, "attention") as c:
        assert OperationCheckpointContext.get_current() is c and c.checkpointing
    assert OperationCheckpointContext.get_current() is None
