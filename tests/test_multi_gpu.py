"""Multi-GPU equivalence cases (fused peer-memory path vs library collectives vs a single-process oracle), launched as
child processes under torch.distributed.run.  Skipped unless the box has at least two GPUs."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                 reason="needs at least two GPUs")]

CASES = Path(__file__).parent / "dist_cases"


def _launch(script, *args, port, nproc=2, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(CASES / script), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def _need(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")


@pytest.mark.parametrize("args,port", [
    (["--comm", "auto"], 29731),                          # fused reduce-scatter + AdamW/all-gather kernels
    (["--comm", "nccl"], 29732),                          # library collectives
    (["--strategy", "FULL_SHARD", "--comm", "fused"], 29733),          # one-sided shard pulls + slot-ring reduce-scatter
    (["--strategy", "FULL_SHARD", "--comm", "fused", "--recompute"], 29734),
    (["--strategy", "FULL_SHARD", "--comm", "fused", "--accum", "2"], 29745),
    (["--strategy", "FULL_SHARD", "--comm", "nccl"], 29746),
    (["--strategy", "NO_SHARD"], 29735),
])
def test_engine_matches_single_process_on_two_gpus(args, port):
    out = _launch("engine_equivalence.py", "--device", "cuda", *args, port=port)
    assert "ok=True" in out
    if "fused" in args:
        assert "fused=True" in out


@pytest.mark.parametrize("nproc", [4, 8])
@pytest.mark.parametrize("args,port", [
    (["--comm", "fused"], 29751),
    (["--strategy", "FULL_SHARD", "--comm", "fused"], 29752),
])
def test_engine_matches_single_process_on_more_gpus(args, port, nproc):
    """The peer-memory reduce-scatter / AdamW-broadcast / shard-pull kernels at 4 and 8 ranks."""
    _need(nproc)
    out = _launch("engine_equivalence.py", "--device", "cuda", *args, port=port + nproc, nproc=nproc)
    assert "ok=True" in out and "fused=True" in out


@pytest.mark.parametrize("args,port", [([], 29736), (["--fused"], 29737)])
def test_tensor_parallel_decoder_on_two_gpus(args, port):
    out = _launch("tp_equivalence.py", "--cuda", *args, port=port)
    assert "ok=False" not in out


@pytest.mark.parametrize("nproc", [4, 8])
def test_fused_tensor_parallel_decoder_on_more_gpus(nproc):
    _need(nproc)
    out = _launch("tp_equivalence.py", "--cuda", "--fused", port=29760 + nproc, nproc=nproc)
    assert "ok=False" not in out


@pytest.mark.parametrize("mode,port", [("sp", 29738), ("pp", 29739), ("cp", 29743), ("ulysses", 29744)])
def test_trainer_config_tensor_sequence_and_pipeline_parallel_on_two_gpus(mode, port):
    """YAML-style config -> SOTATrainer -> tensor + sequence parallel decoder on the fused all-gather->GEMM /
    GEMM->reduce-scatter kernels, a 2-stage pipeline, and context parallelism (ring attention with K/V over peer memory,
    Ulysses all-to-all): losses and the written checkpoint against a single-process trainer."""
    out = _launch("trainer_nd.py", "--mode", mode, "--cuda", port=port)
    assert "RESULT" in out and "ok=True" in out
    if mode == "sp":
        assert "tp comm: fused" in out


def test_weight_gather_gemm_on_two_gpus():
    """The parameter all-gather of a ZeRO-3 forward inside the GEMM kernel equals the product with the full weight."""
    out = _launch("weight_gather_gemm.py", port=29742)
    assert "RESULT weight_gather ok=True" in out


@pytest.mark.parametrize("comm,port", [("nccl", 29741), ("peer", 29742)])
def test_context_parallel_attention_on_two_gpus(comm, port):
    """Causal attention over a sequence sharded on two GPUs == full attention; K/V and dK/dV travel by NCCL send/recv
    or through the framework's peer-memory kernels (pull all-gather, reduce-scatter)."""
    out = _launch("cp_equivalence.py", "--cuda", "--comm", comm, port=port)
    assert out.count("ok=True") == 2
    assert ("path=peer" in out) == (comm == "peer")
    print(out[out.index("TIMING"):].splitlines()[0])


@pytest.mark.parametrize("comm,port", [("fused", 29771), ("nccl", 29772)])
def test_dpo_with_sharded_frozen_reference_on_two_gpus(comm, port):
    """Policy under FULL_SHARD, frozen reference as parameter-only shards pulled layer by layer: losses, gradient norms
    and weights against a single-process run."""
    out = _launch("preference_equivalence.py", "--device", "cuda", "--comm", comm, port=port)
    assert "RESULT preference" in out and "ok=True" in out
    assert ("fused=True" in out) == (comm == "fused")


def test_pipeline_of_tensor_parallel_pairs_on_four_gpus():
    """pp=2 x tp=2 with sequence parallelism through the trainer: fused tensor-parallel GEMMs inside the stages,
    token-sharded activations between them."""
    _need(4)
    out = _launch("trainer_nd.py", "--mode", "tp_pp", "--cuda", port=29781, nproc=4)
    assert "RESULT mode=tp_pp ok=True" in out


@pytest.mark.parametrize("nproc,comm,port", [(2, "auto", 29790), (4, "auto", 29782), (4, "nccl", 29791)])
def test_expert_parallel_trainer(nproc, comm, port):
    """`distributed.parallel.ep: 2` through the trainer on the CUDA kernels (device-side routing, grouped expert
    GEMMs): losses, gradient norms, checkpoint and export against the single-process oracle, with the tokens moved by
    the peer-memory dispatcher (`auto`) or by the library all-to-all (`nccl`)."""
    _need(nproc)
    out = _launch("trainer_nd.py", "--mode", "ep", "--cuda", "--comm", comm, port=port, nproc=nproc)
    assert "RESULT mode=ep ok=True" in out
    used_peer = "ep_peer_calls=0" not in out
    assert used_peer == (comm == "auto"), out[-2000:]


@pytest.mark.parametrize("nproc", [2, 4])
def test_expert_parallel_dispatch_over_peer_memory(nproc):
    """Peer-memory dispatch / combine kernels against the library all-to-all and the all-experts-local block."""
    _need(nproc)
    out = _launch("ep_peer_equivalence.py", port=29782 + nproc, nproc=nproc)
    assert "arm=peer" in out and "ok=False" not in out
