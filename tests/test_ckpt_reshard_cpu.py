"""Optimizer shards of a tensor- / pipeline-parallel run are re-sliced along the data-parallel axis only: shards of
another tp rank or pipeline stage hold other parameters under the same unit names."""
import pytest
import torch

from trainscale_b200.ckpt import reshard_optimizer_state, select_model_parallel_shards
from trainscale_b200.core.errors import CheckpointLoadError


def _shard(tp, pp, dp, tp_size=2, pp_size=1, dp_size=2, numel=8):
    n = numel // dp_size
    base = 1000.0 * tp + 100.0 * pp                 # a value that tells which tp rank / stage a number came from
    vals = base + torch.arange(dp * n, (dp + 1) * n, dtype=torch.float32)
    return {"step": 3, "world": dp_size, "rank": dp, "strategy": "SHARD_GRAD_OP", "param_groups": [],
            "mesh": {"tp": [tp, tp_size], "pp": [pp, pp_size], "dp_cp": [dp, dp_size]},
            "units": {"layers.0": {"master": vals.clone(), "exp_avg": vals * 0.5, "exp_avg_sq": vals * 0.25,
                                   "shard_start": dp * n, "numel": numel}}}


def test_reslice_stays_inside_the_data_parallel_group_of_matching_tp_rank():
    shards = [_shard(tp, 0, dp) for tp in range(2) for dp in range(2)]      # tp 2 x dp 2, file order as globbed
    for tp in range(2):
        mesh = {"tp": [tp, 2], "pp": [0, 1], "dp_cp": [0, 1]}               # resumed as tp 2 x dp 1
        mine = select_model_parallel_shards(shards, mesh)
        assert [s["mesh"]["tp"][0] for s in mine] == [tp, tp] and [s["rank"] for s in mine] == [0, 1]
        out = reshard_optimizer_state(mine, 0, 1, {"layers.0": (8, 0, 8)})
        want = 1000.0 * tp + torch.arange(8, dtype=torch.float32)
        assert torch.equal(out["units"]["layers.0"]["master"], want)
        assert torch.equal(out["units"]["layers.0"]["exp_avg_sq"], want * 0.25)


def test_changed_tensor_or_pipeline_layout_is_refused():
    shards = [_shard(tp, 0, dp) for tp in range(2) for dp in range(2)]
    with pytest.raises(CheckpointLoadError, match="tp=2"):
        select_model_parallel_shards(shards, {"tp": [0, 1], "pp": [0, 1], "dp_cp": [0, 4]})
    with pytest.raises(CheckpointLoadError, match="pp=1"):
        select_model_parallel_shards(shards, {"tp": [0, 2], "pp": [0, 2], "dp_cp": [0, 1]})
    legacy = [dict(s) for s in shards]
    for s in legacy:
        s.pop("mesh")
    with pytest.raises(CheckpointLoadError, match="no mesh coordinates"):
        select_model_parallel_shards(legacy, {"tp": [0, 2], "pp": [0, 1], "dp_cp": [0, 1]})
    with pytest.raises(CheckpointLoadError, match="found 1 optimizer shards"):
        select_model_parallel_shards(shards[:3], {"tp": [1, 2], "pp": [0, 1], "dp_cp": [0, 1]})
