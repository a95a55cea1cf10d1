"""Failure detection and restart, tested on the host (gloo ranks on CPU): lost heartbeats, a rank that leaves, a rank
that raises, a damaged checkpoint, restart at another world size."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

CASE = Path(__file__).parent / "dist_cases" / "fault_cases.py"


def spawn(world, port, *args, timeout=240):
    """Plain child processes (no launcher that would kill the survivors when one rank leaves)."""
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(CASE), *args], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()                      # this exact child
            o, _ = p.communicate()
            o += "\n<timed out>"
        outs.append((p.returncode, o))
    return outs


def test_heartbeat_monitor_with_fake_store():
    from trainscale_b200.parallel.dist_utils import FaultInjector, HeartbeatMonitor

    class Store:                                       # add(key, n) -> new value, like torch's stores
        def __init__(self):
            self.d, self.dropped = {}, set()

        def add(self, k, n):
            if n and k in self.dropped:
                return self.d.get(k, 0)                # the message is lost
            self.d[k] = self.d.get(k, 0) + n
            return self.d[k]

    st = Store()
    mons = [HeartbeatMonitor(st, r, 3) for r in range(3)]
    now = 0.0
    for _ in range(3):
        for m in mons:
            m.beat()
        now += 1.0
        assert mons[0].stale_ranks(2.5, now) == []
    st.dropped.add("hb/1")                             # rank 1's updates stop arriving
    for _ in range(3):
        for m in mons:
            m.beat()
        now += 1.0
        stale = mons[0].stale_ranks(2.5, now)
    assert stale == [1]
    st.dropped.clear()                                 # a slow rank that comes back is no longer stale
    mons[1].beat()
    assert mons[0].stale_ranks(2.5, now + 0.1) == []
    inj = FaultInjector("raise@2:rank1,sleep@1=0.01", rank=1)
    inj.at_step(0)
    inj.at_step(1)
    with pytest.raises(RuntimeError):
        inj.at_step(2)
    FaultInjector("raise@2:rank1", rank=0).at_step(2)  # other ranks are not affected


def test_lost_heartbeats_are_noticed_by_every_rank():
    outs = spawn(3, 29761, "--mode", "heartbeat")
    assert all(rc == 0 for rc, _ in outs), outs
    assert all("detected=(" in o and "[2]" in o for _, o in outs)


def test_a_rank_that_leaves_ends_the_next_collective_with_an_error():
    outs = spawn(2, 29762, "--mode", "exit")
    assert outs[1][0] == 17                            # the rank that left
    assert outs[0][0] == 3 and "collective failed at step 2" in outs[0][1], outs[0]


def test_restart_from_latest_undamaged_checkpoint_at_another_world_size(tmp_path):
    from trainscale_b200.ckpt import find_latest_valid_checkpoint, list_checkpoints, verify_checkpoint
    outs = spawn(2, 29763, "--mode", "train", "--out", str(tmp_path), "--fault", "raise@3:rank1")
    assert outs[1][0] == 5 and "died" in outs[1][1]
    assert outs[0][0] != 0                             # the survivor's collective failed (or timed out)
    cks = list_checkpoints(tmp_path)
    assert [c.name for c in cks][:3] == ["checkpoint-1", "checkpoint-2", "checkpoint-3"]
    # damage the newest complete one: a truncated optimizer shard and a flipped byte in the weights
    newest = find_latest_valid_checkpoint(tmp_path)
    shard = sorted((newest / "optim").glob("shard-*.pt"))[0]
    shard.write_bytes(shard.read_bytes()[: shard.stat().st_size // 2])
    assert any("truncated" in p for p in verify_checkpoint(newest))
    older = list_checkpoints(tmp_path)[-2] if newest == cks[-1] else cks[-1]
    assert find_latest_valid_checkpoint(tmp_path) != newest
    w = next(newest.glob("*.safetensors"))
    raw = bytearray(w.read_bytes())
    raw[-1] ^= 0xFF
    w.write_bytes(bytes(raw))
    assert any("sha256" in p for p in verify_checkpoint(newest))
    # restart as ONE process: optimizer shards written by two ranks are re-sliced
    outs = spawn(1, 29764, "--mode", "resume", "--out", str(tmp_path))
    assert outs[0][0] == 0, outs[0][1][-3000:]
    assert "ok=True" in outs[0][1] and "skipped=" in outs[0][1] and "skipped=0" not in outs[0][1]
    del older


def test_expired_peer_wait_skips_the_update_and_raises(tmp_path):
    """A fused collective that gave up waiting for a peer sets the heap's status word.  The engine folds that word into
    its skip flag on the device (no update from an unwritten gradient shard) and the trainer raises where it reads the
    loss.  The failing call is faked on the host: a status word that the test sets."""
    import pytest
    import torch
    from trainscale_b200.core.errors import CommunicationError
    from trainscale_b200.parallel.symm import SymmetricHeap
    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.trainer.sota_trainer import SOTATrainer

    cfg = SOTAConfig.from_dict({
        "model": {"architecture": {"vocab_size": 128, "hidden_size": 32, "intermediate_size": 64, "num_hidden_layers": 1,
                                   "num_attention_heads": 2, "num_key_value_heads": 1}},
        "optimizer": {"type": "adamw", "learning_rate": 1e-2}, "scheduler": {"type": "constant", "warmup_steps": 0},
        "distributed": {"enabled": False, "strategy": "ddp"}, "hardware": {"device": "cpu", "precision": "fp32"},
        "data": {"max_seq_length": 16},
        "training": {"output_dir": str(tmp_path), "max_steps": 4, "save_strategy": "no", "eval_strategy": "no"}})
    tr = SOTATrainer(cfg)
    tr.setup_model()
    heap = SymmetricHeap.__new__(SymmetricHeap)          # the status word and its readers, without any peer memory
    heap.status = torch.zeros(1, dtype=torch.int32)
    heap.rank, heap.world = 0, 1
    tr.engine._symm = heap
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(0))
    tr.train_step({"input_ids": ids, "labels": ids})       # healthy step: weights move
    before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    heap.status.fill_(1)                                   # "a peer did not arrive"
    with pytest.raises(CommunicationError):
        tr.train_step({"input_ids": ids, "labels": ids})
    for n, p in tr.model.named_parameters():
        assert torch.equal(p.detach(), before[n]), f"{n} was updated from an unreduced gradient"
    assert int(heap.status) == 0                           # reading the status clears it
    tr.train_step({"input_ids": ids, "labels": ids})
    assert any(not torch.equal(p.detach(), before[n]) for n, p in tr.model.named_parameters())
