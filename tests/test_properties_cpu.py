"""Property tests (hypothesis).  Pipeline schedules: for any stage / micro-batch count every generator emits each
operation exactly once per (stage, micro-batch), the per-stage orders are executable without deadlock and memory limits
are kept.  Context-parallel layouts partition the sequence and invert; mesh coordinates round-trip; optimizer shards
re-slice exactly between any two world sizes."""
import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st      # noqa: E402

from trainscale_b200.parallel import pp as PP                 # noqa: E402
from trainscale_b200.parallel import pipeline as PL           # noqa: E402
from trainscale_b200.parallel import zbpp as Z                # noqa: E402


@settings(max_examples=60, deadline=None)
@given(P=st.integers(1, 8), extra=st.integers(0, 12), name=st.sampled_from(["gpipe", "1f1b", "zero_bubble"]))
def test_closed_form_schedules_are_complete_and_deadlock_free(P, extra, name):
    M = P + extra
    lists = [PP.create_schedule(name, s, P, M) for s in range(P)]
    for lst in lists:
        for op in ("F", "B") + (("W",) if name == "zero_bubble" else ()):
            assert sorted(a.mb for a in lst if a.op == op) == list(range(M))
        pos = {(a.op, a.mb): i for i, a in enumerate(lst)}
        assert all(pos[("B", m)] > pos[("F", m)] for m in range(M))
        if name == "zero_bubble":
            assert all(pos[("W", m)] > pos[("B", m)] for m in range(M))
    r = PP.simulate(lists)                                   # raises on a deadlock
    assert 0.0 <= r["bubble_fraction"] < 1.0
    if name != "gpipe" and P > 1:
        # in-flight activations of 1F1B-type orders never exceed P - stage (W releases them under zero-bubble)
        for s, lst in enumerate(lists):
            live = peak = 0
            for a in lst:
                live += 1 if a.op == "F" else -1 if a.op == ("W" if name == "zero_bubble" else "B") else 0
                peak = max(peak, live)
            assert peak <= (P - s) + (P if name == "zero_bubble" else 0)


@settings(max_examples=30, deadline=None)
@given(P=st.integers(1, 4), V=st.integers(2, 3), groups=st.integers(1, 3))
def test_interleaved_schedule_covers_every_chunk(P, V, groups):
    M = P * groups
    for s in range(P):
        lst = PP.interleaved_1f1b_schedule(s, P, M, V)
        for c in range(V):
            assert sorted(a.mb for a in lst if a.op == "F" and a.chunk == c) == list(range(M))
            assert sorted(a.mb for a in lst if a.op == "B" and a.chunk == c) == list(range(M))


@settings(max_examples=25, deadline=None)
@given(half_p=st.integers(1, 4), half_m=st.integers(1, 8))
def test_chimera_order_is_complete_and_ordered(half_p, half_m):
    P, M = 2 * half_p, 2 * half_m
    lists = PL.chimera_schedule(P, M)
    assert len(lists) == P
    for w, lst in enumerate(lists):
        down = [a for a in lst if a.chunk == 0]
        up = [a for a in lst if a.chunk == 1]
        assert sorted(a.mb for a in down if a.op == "F") == list(range(M // 2))
        assert sorted(a.mb for a in up if a.op == "F") == list(range(M // 2, M))
        pos = {(a.op, a.mb): i for i, a in enumerate(lst)}
        assert all(pos[("B", m)] > pos[("F", m)] for m in range(M))


@settings(max_examples=40, deadline=None)
@given(P=st.integers(2, 6), extra=st.integers(0, 8), f=st.floats(50, 200), b=st.floats(50, 200), w=st.floats(50, 200),
       slack=st.integers(1, 6), h2=st.booleans())
def test_cost_driven_zero_bubble_scheduler(P, extra, f, b, w, slack, h2):
    M = P + extra
    act, par = 1 << 20, 1 << 22
    prof = [Z.StageProfile(f, b, w, act, par, 0.0, 0.0) for _ in range(P)]
    limit = par + slack * act
    r = Z.ZBPPScheduleOptimizer(Z.ScheduleConfig(P, M, limit, prof, enable_interleaving=not h2)).optimize()
    assert all(v <= limit for v in r.peak_memory_bytes.values())
    for s, lst in r.schedule.items():
        for op in (Z.OpType.FORWARD, Z.OpType.BACKWARD_INPUT, Z.OpType.BACKWARD_PARAMS):
            assert sorted(x.microbatch_id for x in lst if x.op_type == op) == list(range(M))
        starts = [x.start_us for x in lst]
        assert starts == sorted(starts)
    acts = r.actions()
    PP.simulate(acts, {"F": f, "B": b, "W": w})              # executable in the emitted order
    if slack >= P:       # with 1F1B's memory available the result is never slower than 1F1B
        base = PP.simulate([PP.one_f_one_b_schedule(s, P, M) for s in range(P)], {"F": f, "B": b + w, "W": 0.0})
        assert r.makespan_us <= base["makespan"] * (1 + 1e-9) + 1e-6


@settings(max_examples=40, deadline=None)
@given(cp=st.integers(1, 8), mult=st.integers(1, 4), name=st.sampled_from(["head_tail", "zigzag", "ptrr"]))
def test_context_parallel_layouts_partition_the_sequence(cp, mult, name):
    import torch
    from trainscale_b200.parallel import cp as CP
    S = 2 * cp * mult * 4
    x = torch.arange(S).view(1, S, 1)
    parts = [CP.create_balancer(name, cp, r).shard(x) for r in range(cp)]
    assert sorted(torch.cat(parts, 1).flatten().tolist()) == list(range(S))          # every token exactly once
    assert len({p.shape[1] for p in parts}) == 1                                      # equal shares
    torch.testing.assert_close(CP.create_balancer(name, cp, 0).unshard(parts), x)    # and the inverse restores order
    if name == "head_tail" and cp > 1:
        # causal work (sum of positions + 1) is balanced to within one chunk pair
        work = [int((p.flatten() + 1).sum()) for p in parts]
        assert max(work) - min(work) <= S


@settings(max_examples=40, deadline=None)
@given(pp=st.integers(1, 3), rep=st.integers(1, 2), shard=st.integers(1, 3), cpd=st.integers(1, 2), tp=st.integers(1, 2))
def test_mesh_coordinates_round_trip(pp, rep, shard, cpd, tp):
    from trainscale_b200.parallel.mesh import ParallelDims, ParallelDimsConfig
    world = pp * rep * shard * cpd * tp
    cfg = ParallelDimsConfig(dp_replicate=rep, dp_shard=shard, cp=cpd, tp=tp, pp=pp, world_size=world)
    seen = set()
    for r in range(world):
        d = ParallelDims(cfg, rank=r, create_groups=False)
        assert d.rank_of(**d.coords) == r
        seen.add(tuple(sorted(d.coords.items())))
        tp_ranks = d.ranks_along(("tp",))
        assert r in tp_ranks and len(tp_ranks) == tp and max(tp_ranks) - min(tp_ranks) == tp - 1   # tp innermost
        assert d.size("fsdp") == shard * cpd and d.size("loss") == rep * shard * cpd
    assert len(seen) == world


@settings(max_examples=30, deadline=None)
@given(old=st.integers(1, 6), new=st.integers(1, 6), used=st.integers(1, 5000))
def test_optimizer_shards_reslice_exactly_between_world_sizes(old, new, used):
    import torch
    from trainscale_b200.ckpt import reshard_optimizer_state
    align = 64

    def padded(world):
        q = align * world
        return (used + q - 1) // q * q

    full = torch.arange(used, dtype=torch.float32)
    n_old = padded(old)
    buf = torch.cat((full, torch.zeros(n_old - used)))
    shards = [{"rank": r, "world": old, "step": 3,
               "units": {"u": {"master": buf[r * n_old // old:(r + 1) * n_old // old].clone(),
                               "exp_avg": buf[r * n_old // old:(r + 1) * n_old // old].clone() * 2, "exp_avg_sq": None,
                               "shard_start": r * n_old // old, "numel": n_old}}} for r in range(old)]
    n_new = padded(new)
    got = []
    for r in range(new):
        layout = {"u": (n_new, r * n_new // new, n_new // new)}
        out = reshard_optimizer_state(shards, r, new, layout)
        assert out["units"]["u"]["exp_avg_sq"] is None and out["step"] == 3
        got.append(out["units"]["u"]["master"])
        torch.testing.assert_close(out["units"]["u"]["exp_avg"], out["units"]["u"]["master"] * 2)
    whole = torch.cat(got)
    assert whole.numel() == n_new
    torch.testing.assert_close(whole[:used], full)
    assert float(whole[used:].abs().sum()) == 0.0
