"""gloo / CPU multi-process tests of the flat engine's sharding, reduction and re-gather logic."""
import subprocess
import sys
from pathlib import Path

import pytest

CASE = Path(__file__).parent / "dist_cases" / "engine_equivalence.py"


def launch(nproc, *args, port=29611, timeout=300):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(CASE), *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("strategy,port", [("SHARD_GRAD_OP", 29611), ("NO_SHARD", 29612), ("FULL_SHARD", 29613)])
def test_two_rank_engine_matches_single_process(strategy, port):
    r = launch(2, "--device", "cpu", "--strategy", strategy, port=port)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("extra,port", [(["--recompute"], 29614), (["--accum", "2"], 29615)])
def test_full_shard_with_recompute_and_accumulation(extra, port):
    """FULL_SHARD re-gathers inside the recomputation of a layer and reduces every micro-batch into its shard."""
    r = launch(2, "--device", "cpu", "--strategy", "FULL_SHARD", *extra, port=port)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ok=True" in r.stdout


def test_tensor_and_sequence_parallel_match_unsharded():
    case = Path(__file__).parent / "dist_cases" / "tp_equivalence.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29631", str(case)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == 2


def test_pipeline_stages_match_single_process():
    case = Path(__file__).parent / "dist_cases" / "pp_equivalence.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29651", str(case)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == 6


def test_schedule_simulator_bubbles():
    from trainscale_b200.parallel.pp import create_schedule, simulate
    P, M = 4, 8
    res = {n: simulate([create_schedule(n, s, P, M) for s in range(P)]) for n in ("gpipe", "1f1b", "zero_bubble")}
    assert abs(res["1f1b"]["bubble_fraction"] - (P - 1) / (M + P - 1)) < 1e-9
    assert res["zero_bubble"]["bubble_fraction"] < 0.5 * res["1f1b"]["bubble_fraction"]
    assert res["gpipe"]["makespan"] == res["1f1b"]["makespan"]


@pytest.mark.parametrize("n,port", [(2, 29671), (4, 29672)])
def test_ring_attention_matches_full_attention(n, port):
    case = Path(__file__).parent / "dist_cases" / "cp_equivalence.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(case)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == n


def test_head_tail_and_zigzag_layouts_roundtrip():
    import torch
    from trainscale_b200.parallel.cp import HeadTailBalancer, ZigZagBalancer, shard_inputs
    x = torch.arange(2 * 32).view(2, 32)
    for cls in (HeadTailBalancer, ZigZagBalancer):
        parts = [cls(4, r).shard(x) for r in range(4)]
        assert torch.equal(cls(4, 0).unshard(parts), x)
    b = shard_inputs({"input_ids": x}, 4, 1)
    assert b["position_ids"][0].tolist() == list(range(4, 8)) + list(range(24, 28))
    assert b["labels"][0, 3].item() == x[0, 8].item() and b["labels"][0, -1].item() == x[0, 28].item()


def test_expert_parallel_moe_matches_local_moe():
    case = Path(__file__).parent / "dist_cases" / "ep_equivalence.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29682", str(case)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == 2


def test_hybrid_sharding_four_ranks():
    """2 shard groups x 2 replicas: reduce-scatter inside a group, average of the shards across groups."""
    r = launch(4, "--device", "cpu", "--strategy", "SHARD_GRAD_OP", "--replicate", "2", port=29616)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


ND_CASE = Path(__file__).parent / "dist_cases" / "trainer_nd.py"


@pytest.mark.parametrize("mode,port", [("pp", 29621), ("sp", 29622), ("cp", 29623), ("ulysses", 29624)])
def test_trainer_config_drives_pipeline_and_sequence_parallel(mode, port):
    """SOTATrainer with `distributed.strategy: pipeline` (1F1B, 2 micro-batches), with tensor + sequence parallelism and
    with context parallelism (ring attention on head-tail shards, or all-to-all head / sequence exchange on contiguous
    shards) reproduces the single-process losses step by step (global grad-norm clip included) and writes a checkpoint
    equal to the single-process weights."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ND_CASE), "--mode", mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_tensor_parallel_pairs_times_data_parallel_clip_norm():
    """tp=2 x dp=2 on four gloo ranks: the global gradient norm (replicated parameters counted once) and the losses
    equal the single-process trainer's."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29625", str(ND_CASE), "--mode", "tp_dp"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT mode=tp_dp ok=True" in r.stdout


def test_pipeline_stages_of_tensor_parallel_pairs_with_sequence_parallelism():
    """pp=2 x tp=2 (+ sequence parallelism) on four gloo ranks reproduces the single-process losses and checkpoint."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29626", str(ND_CASE), "--mode", "tp_pp"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT mode=tp_pp ok=True" in r.stdout


def test_expert_parallelism_from_the_config_matches_single_process():
    """`distributed.parallel.ep: 2` on four gloo ranks (two expert-parallel pairs x two replicas of every expert):
    losses, the one global gradient norm both engines clip with, the HuggingFace-layout checkpoint (experts gathered)
    and a resume, against the single-process trainer on the same mixture-of-experts decoder."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29627", str(ND_CASE), "--mode", "ep"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT mode=ep ok=True" in r.stdout
