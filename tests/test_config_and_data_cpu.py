"""Config schema, Result type, tokenizer, prompt engine stages, length manager, packing, collate, DataPipeline."""
import os
import pytest
import torch
import yaml

from trainscale_b200.config.data_schema import (FIMConfig, PackingConfig, PackingStrategy, SpanCorruptionConfig,
                                                load_config, load_config_dict)
from trainscale_b200.config.sota_config import SOTAConfig, get_full_finetune_preset, get_qlora_preset
from trainscale_b200.core import Err, Ok, flat_map, is_err, is_ok, map_err, map_result, unwrap_or
from trainscale_b200.core.errors import SchemaValidationError, TemplateRenderError
from trainscale_b200.data import prompt_engine as PE
from trainscale_b200.data.collate import create_causal_lm_collate, create_collate_fn
from trainscale_b200.data.dataloader_factory import build_distributed_dataloaders
from trainscale_b200.data.length_manager import (create_content_distributor, create_dynamic_collate_fn,
                                                 create_length_manager, smart_truncate)
from trainscale_b200.data.packing import (create_packed_attention_mask, cu_seqlens_from_document_ids,
                                          first_fit_decreasing, get_packing_stats, pack_sequences, unpack_sequences)
from trainscale_b200.data.pipeline import DataPipeline
from trainscale_b200.data.tokenization import create_tokenizer

BASE = {"type": "data_module", "version": "1.0", "dataset": {"name": "mem"}, "tokenizer": {"name_or_path": "byte", "max_length": 64}}


def test_result_helpers():
    assert is_ok(Ok(1)) and is_err(Err("x"))
    assert map_result(Ok(2), lambda v: v + 1) == Ok(3) and map_result(Err("e"), lambda v: v) == Err("e")
    assert flat_map(Ok(2), lambda v: Err("bad")) == Err("bad")
    assert map_err(Err("e"), str.upper) == Err("E") and unwrap_or(Err("e"), 7) == 7
    with pytest.raises(ValueError):
        Err("plain").unwrap()


def test_data_schema_validation(tmp_path):
    assert load_config_dict(BASE).is_ok()
    bad = dict(BASE, type="nope")
    r = load_config_dict(bad)
    assert r.is_err() and isinstance(r.error, SchemaValidationError)
    assert load_config_dict({k: v for k, v in BASE.items() if k != "tokenizer"}).is_err()
    p = tmp_path / "c.yaml"
    p.write_text(yaml.safe_dump(dict(BASE, training_mode="full", optimizer={"type": "lion"})))
    assert load_config(p).is_ok()                       # training keys are ignored by the data loader ...
    assert SOTAConfig.from_yaml(p).optimizer.type.value == "lion"   # ... and data keys by the training loader
    assert load_config(tmp_path / "missing.yaml").is_err()


def test_sota_config_strict_sections_and_roundtrip(tmp_path):
    with pytest.raises(TypeError):
        SOTAConfig.from_dict({"scheduler": {"nonexistent": 1}})
    c = SOTAConfig.from_dict({"training_mode": "qlora", "distributed": {"strategy": "fsdp2", "parallel": {"tp": 2, "pp": 2}}})
    assert c.lora.enabled and c.quantization.load_in_4bit and c.distributed.parallel.pp == 2
    c.save_yaml(tmp_path / "o.yaml")
    assert SOTAConfig.from_yaml(tmp_path / "o.yaml").to_dict() == c.to_dict()
    assert get_qlora_preset("m").training_mode.value == "qlora" and not get_full_finetune_preset().lora.enabled
    with pytest.raises(ValueError):
        SOTAConfig.from_dict({"training": {"gradient_accumulation_steps": 0}})


def test_tokenizer_wrapper_roundtrip_and_special_tokens():
    t = create_tokenizer(name_or_path="byte", max_length=16)
    e = t.encode("héllo")
    assert len(e.input_ids) == 16 and sum(e.attention_mask) == 7
    assert t.decode(e.input_ids) == "héllo"
    assert t.add_special_tokens_dict({"additional_special_tokens": ["<x>"]}) == 1 and t.vocab_growth == 1
    assert t.encode_raw("a<x>b") == [97, 260, 98]
    assert t.get_special_tokens_mask([257, 97, 256]) == [1, 0, 1]


def test_prompt_engine_sft_masks_prompt_and_keeps_answer():
    t = create_tokenizer(name_or_path="byte", max_length=128)
    e = PE.create_finetuning_engine(t, 128, "completion")
    x = e.process({"prompt": "Q: 2+2? A: ", "completion": "4"})
    trained = [l for l in x.labels if l != -100]
    assert trained == [ord("4"), t.eos_token_id] and x.labels[:x.extras["prompt_length"]] == [-100] * x.extras["prompt_length"]
    long = e.process({"prompt": "p" * 500, "completion": "answer"})
    assert t.decode([l for l in long.labels if l != -100]) == "answer"       # the prompt is trimmed, never the answer
    mt = PE.create_finetuning_engine(t, 128, "multi_turn").process(
        {"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]})
    assert t.decode([l for l in mt.labels if l != -100]).strip() == "yo"
    with pytest.raises(TemplateRenderError):
        PE.render_template("{missing}", {})


def test_prompt_engine_pretraining_variants_and_packing():
    t = create_tokenizer(name_or_path="byte", max_length=64)
    fim = PE.create_pretraining_engine(t, 64, "fill_in_middle", fim=FIMConfig(enabled=True, fim_rate=1.0))
    s = t.decode(fim.process({"text": "def f(x): return x"}).input_ids, skip_special_tokens=False)
    assert "<fim_prefix>" in s and "<fim_suffix>" in s and "<fim_middle>" in s
    sc = PE.create_pretraining_engine(t, 64, "span_corruption", span_corruption=SpanCorruptionConfig(enabled=True))
    x = sc.process({"text": "the quick brown fox jumps over the lazy dog"})
    assert x.extras["num_spans"] >= 1 and any(l != -100 for l in x.labels)
    pk = PE.create_pretraining_engine(t, 32, packing=PackingConfig(enabled=True, strategy=PackingStrategy.FFD))
    packs = pk.pack_documents(["aaaa", "bb", "c" * 20, "d" * 50])
    for p in packs:
        assert len(p.input_ids) == 32 and p.cu_seqlens[0] == 0
        for a, b in zip(p.cu_seqlens[:-1], p.cu_seqlens[1:]):      # positions restart per document
            assert p.position_ids[a:b] == list(range(b - a)) and len(set(p.document_ids[a:b])) == 1
        assert all(d == -1 for d in p.document_ids[p.cu_seqlens[-1]:])


def test_prompt_engine_preference_stages():
    t = create_tokenizer(name_or_path="byte", max_length=48)
    d = PE.create_rl_engine(t, 48, "dpo").process({"prompt": "Q", "chosen": "good", "rejected": "bad"})
    assert len(d.chosen_input_ids) == len(d.rejected_input_ids) == 48
    assert t.decode([l for l in d.chosen_labels if l != -100]) == "good"
    k = PE.create_rl_engine(t, 48, "kto", undesirable_weight=0.5).process({"prompt": "Q", "response": "r", "label": False})
    assert k.kto_tag is False and k.weight == 0.5
    g = PE.create_rl_engine(t, 48, "grpo").process({"prompt": "Q", "responses": ["a", "bb", "ccc"], "scores": [1, 0, 2]})
    assert len(g.responses_input_ids) == 3 and g.scores == [1.0, 0.0, 2.0]
    p = PE.create_rl_engine(t, 16, "ppo").process({"prompt": "abc"})
    assert p.query_attention_mask[-3:] == [1, 1, 1] and p.query_attention_mask[0] == 0      # left padded
    b = PE.batch_to_dict([d, d])
    assert b["chosen_input_ids"].shape == (2, 48)


def test_length_manager_truncation_and_budgets():
    text = "First sentence here. Second one, with a clause; and more words to follow after that point. Third."
    assert smart_truncate(text, 60).endswith(";") and len(smart_truncate(text, 60)) <= 60
    assert smart_truncate(text, 30, "left") == text[-30:] and len(smart_truncate(text, 30, "middle")) == 30
    d = create_content_distributor("adaptive", 100, label_columns=["out"])
    a = d.allocate({"inp": 300, "out": 80})
    assert sum(a.values()) <= 90 and a["out"] >= 54            # labels keep at least 60 % of the budget
    assert create_content_distributor("equal", 110).allocate({"a": 500, "b": 500}) == {"a": 50, "b": 50}
    pr = create_content_distributor("priority", 110, priorities={"a": 0, "b": 1}).allocate({"a": 80, "b": 80})
    assert pr == {"a": 80, "b": 20}
    assert create_length_manager(512, "bucket").get_effective_max_length([100, 130]) == 256
    assert create_length_manager(512, "power_of_two").get_effective_max_length([100, 257]) == 512
    assert create_length_manager(512, "longest").get_effective_max_length([100, 130]) == 130
    col = create_dynamic_collate_fn(create_length_manager(64, "bucket", bucket_boundaries=(8, 16, 32, 64)), 0)
    b = col([{"input_ids": torch.arange(1, 11), "attention_mask": torch.ones(10, dtype=torch.long), "labels": torch.arange(1, 11)},
             {"input_ids": torch.arange(1, 6), "attention_mask": torch.ones(5, dtype=torch.long), "labels": torch.arange(1, 6)}])
    assert b["input_ids"].shape == (2, 16) and b["labels"][1, 5:].eq(-100).all()


def test_trainer_side_packing_and_masks():
    bins = first_fit_decreasing([5, 4, 3, 3, 1], 8)
    assert sorted(sum(([5, 4, 3, 3, 1][i] for i in b)) for b in bins) == [8, 8]
    seqs = [{"input_ids": torch.arange(n)} for n in (5, 3, 4, 2)]
    packed = pack_sequences(seqs, 8)
    assert all(p["input_ids"].shape == (8,) for p in packed)
    p0 = packed[0]
    parts = unpack_sequences(p0["input_ids"], p0["cu_seqlens"])
    assert [len(x) for x in parts] == [p0["cu_seqlens"][i + 1] - p0["cu_seqlens"][i] for i in range(len(parts))]
    m = create_packed_attention_mask(torch.tensor([0, 3, 5]), 6)
    assert m[1, 0] == 0 and m[0, 1] == float("-inf") and m[3, 2] == float("-inf") and m[5, 5] == float("-inf")
    cu, mx = cu_seqlens_from_document_ids(torch.tensor([[0, 0, 1, 1, 1, -1], [0, 0, 0, 0, 1, 1]]))
    assert cu.tolist() == [0, 2, 5, 6, 10, 12] and mx == 4
    assert get_packing_stats([5, 4, 3, 3, 1], 8)["efficiency"] == 1.0


def test_collate_and_distributed_loaders():
    c = create_collate_fn(pad_token_id=9)
    b = c([{"input_ids": torch.tensor([1, 2, 3]), "attention_mask": torch.tensor([1, 1, 1]), "labels": torch.tensor([1, 2, 3])},
           {"input_ids": torch.tensor([4]), "attention_mask": torch.tensor([1]), "labels": torch.tensor([4])}])
    assert b["input_ids"][1].tolist() == [4, 9, 9] and b["labels"][1].tolist() == [4, -100, -100]
    s = create_causal_lm_collate(0, shift_labels=True)([{"input_ids": torch.tensor([1, 2, 3])}])
    assert s["labels"].tolist() == [[2, 3, -100]]
    ds = [{"input_ids": torch.tensor([i])} for i in range(10)]
    loaders = build_distributed_dataloaders(ds, 2, batch_size=1, collate_fn=create_collate_fn())
    seen = [sorted(int(b["input_ids"]) for b in dl) for dl in loaders]
    assert sorted(seen[0] + seen[1]) == list(range(10)) and not set(seen[0]) & set(seen[1])


def test_data_pipeline_end_to_end_in_memory():
    raw = dict(BASE, dataset={"name": "mem", "splits": {"train": {"name": "train", "sample_size": 6}}},
               prompt_engine={"stage": "fine_tuning", "max_length": 64, "fine_tuning": {"format": "instruction"}},
               dataloader={"batch_size": 2, "shuffle": False, "pin_memory": False})
    p = DataPipeline.from_config(raw).unwrap()
    p.register_dataset("train", [{"instruction": f"add {i}", "input": "", "output": str(i)} for i in range(10)])
    assert p.discover().unwrap().columns.keys() >= {"instruction", "output"}
    dl = p.get_dataloader("train").unwrap()
    assert len(dl) == 3
    b = next(iter(dl))
    assert b["input_ids"].shape == (2, 64) and (b["labels"] != -100).sum() > 0
    assert DataPipeline.from_config(dict(raw, type="x")).is_err()
    assert p.get_dataloader("nope").is_err()


def test_every_shipped_yaml_parses_and_resolves_its_mesh():
    import glob
    from pathlib import Path
    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.parallel.mesh import create_parallel_dims_from_config
    from trainscale_b200.trainer.sota_trainer import STRATEGY_ALIASES
    files = sorted(glob.glob(str(Path(__file__).resolve().parents[1] / "configs" / "*.yaml")))
    assert len(files) >= 7
    seen = {}
    for f in files:
        c = SOTAConfig.from_yaml(f)
        assert c.distributed.strategy in STRATEGY_ALIASES, f
        if c.distributed.enabled:
            d = create_parallel_dims_from_config(c.distributed, world_size=c.distributed.world_size, rank=0)
            seen[Path(f).name] = d.sizes
    assert seen["llama3_70b_tp4_pp2_fp8.yaml"]["tp"] == 4 and seen["llama3_70b_tp4_pp2_fp8.yaml"]["pp"] == 2
    assert seen["llama3_8b_cp8_128k.yaml"]["cp"] == 8


def _reference_example_yamls():
    from pathlib import Path
    here = Path(__file__).resolve().parent.parent
    # the reference as installed for the comparison arm of bench.py, or a checkout named by TRAINSCALE_REFERENCE
    roots = [here / "baseline" / "_ref" / "data_pipeline" / "examples"]
    if os.environ.get("TRAINSCALE_REFERENCE"):
        roots.append(Path(os.environ["TRAINSCALE_REFERENCE"]) / "data_pipeline" / "examples")
    for root in roots:
        found = sorted(root.glob("*.yaml")) if root.is_dir() else []
        if found:
            return found
    return []


@pytest.mark.parametrize("path", _reference_example_yamls() or [None], ids=lambda p: p.name if p else "absent")
def test_reference_example_yamls_load_through_both_loaders(path):
    """Every example YAML shipped with the reference (data_pipeline/examples/*.yaml) must load, unmodified, through
    the trainer-side loader and the data-side loader, as the reference reads one file twice."""
    if path is None:
        pytest.skip("the reference's example YAMLs are not on this machine")
    cfg = SOTAConfig.from_yaml(path)
    raw = yaml.safe_load(path.read_text())
    if "export" in raw and "save_merged_16bit" in raw["export"]:
        assert cfg.export.save_merged_16bit == raw["export"]["save_merged_16bit"]
    assert cfg.optimizer.learning_rate == float(raw.get("optimizer", {}).get("learning_rate", cfg.optimizer.learning_rate))
    r = load_config(path)
    assert r.is_ok(), r
    assert r.unwrap().tokenizer.name_or_path


def test_the_reference_example_configurations_load():
    """Every example YAML shipped with the reference loads with the loader of its own type: trainer configurations
    (`config_type` / `training_mode` at the top) as `SOTAConfig`, data-pipeline configurations (`type`, `version`,
    `dataset`) through `load_config`, and the flat training-arguments file through `load_training_config`."""
    import glob
    import os
    from pathlib import Path

    import yaml as _yaml
    from trainscale_b200.config.data_schema import load_config
    from trainscale_b200.config.sota_config import SOTAConfig
    from trainscale_b200.config.training_args import load_training_config

    here = Path(__file__).resolve().parents[1]
    roots = [here / "baseline" / "_ref" / "data_pipeline" / "examples",
             Path(os.environ.get("TRAINSCALE_REFERENCE", "/nonexistent")) / "data_pipeline" / "examples"]
    root = next((r for r in roots if r.is_dir()), roots[0])
    files = sorted(glob.glob(str(root / "**" / "*.yaml"), recursive=True))
    if not files:
        pytest.skip("the reference's examples are not on this machine")
    seen = {"sota": 0, "data": 0, "args": 0}
    for f in files:
        top = _yaml.safe_load(open(f))
        if "training_mode" in top or "config_type" in top:
            cfg = SOTAConfig.from_yaml(f)
            assert cfg.model.name_or_path or cfg.model.architecture is not None, f
            seen["sota"] += 1
        if "dataset" in top and "type" in top:
            assert load_config(f).is_ok(), f
            seen["data"] += 1
        if "dataset" not in top and "training" in top and "training_mode" not in top:
            assert load_training_config(f).output_dir, f
            seen["args"] += 1
    assert seen["sota"] >= 5 and seen["data"] >= 8 and seen["args"] >= 1, seen
