"""DataPipeline: one YAML -> tokenizer, prompt engine, datasets and DataLoaders.

After data_pipeline/pipeline.py:81-571: `DataPipeline.from_config(path, token, trust_remote_code) -> Result`, lazy
tokenizer / prompt engine (with a PROPORTIONAL TokenAwareContentDistributor), `discover`, `load_dataset`,
`get_preprocessed_dataset`, `get_dataloader(split, batch_size, distributed, rank, world_size) -> Result[DataLoader]`,
`get_splits`, `create_pipeline`.  Datasets resolve in this order: in-memory data registered with
`register_dataset`, a local file / directory (`dataset.path` or an existing `dataset.name`), the built-in
`synthetic` dataset (uniform random tokens with document boundaries), then the HuggingFace hub.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Any, Mapping, Sequence

from ..config.data_schema import (ContentDistributionMode, PipelineConfig, PromptEngineConfig, TrainingStage,
                                  load_config, load_config_dict)
from ..core.errors import DataLoadingError, DatasetNotFoundError, PipelineError, SplitNotFoundError
from ..core.types import Err, Ok, Result
from ..utils.refargs import ANY, reference_kwargs
from ..introspection import ColumnMapper, DatasetIntrospector
from .collate import create_collate_fn
from .dataloader_factory import build_dataloader
from .dataset_wrappers import create_preprocessed_dataset
from .length_manager import TokenAwareContentDistributor
from .prompt_engine import PromptEngine
from .tokenization import create_tokenizer


class DataPipeline:
    def __init__(self, config: PipelineConfig | None = None, token: str | None = None, trust_remote_code: bool = False, *,
                 dataset_name: str | None = None, dataset_config=None, tokenizer=None, tokenizer_config=None,
                 prompt_template=None, output_schema=None, dataloader_config=None, pipeline_config=None):
        """From a full `PipelineConfig` (`config` / `pipeline_config`), or assembled from parts the way the reference's
        constructor takes them (data_pipeline/pipeline.py:107-160): a dataset name or `DatasetConfig`, a ready tokenizer
        or a `TokenizerConfig`, a `PromptTemplate`, an `OutputSchema`, a `DataLoaderConfig`."""
        config = config if config is not None else pipeline_config
        if isinstance(config, str):                         # DataPipeline("org/dataset", ...): the shorthand
            dataset_name, config = config, None
        if config is None:
            from ..config.data_schema import DataLoaderConfig, DatasetConfig, OutputSchema, PromptTemplate, TokenizerConfig
            if dataset_config is None and dataset_name is None:
                raise ValueError("DataPipeline needs a PipelineConfig, a dataset_config or a dataset_name")
            name = getattr(tokenizer, "name_or_path", None) or "byte"
            config = PipelineConfig(
                "data_module", "1.0", dataset_config if dataset_config is not None else DatasetConfig(dataset_name),
                tokenizer_config if tokenizer_config is not None else TokenizerConfig(name),
                prompt_template if prompt_template is not None else PromptTemplate(),
                None, output_schema if output_schema is not None else OutputSchema(),
                dataloader_config if dataloader_config is not None else DataLoaderConfig())
        self.config = config
        self.token = token or os.environ.get("HF_TOKEN")
        self.trust_remote_code = trust_remote_code
        self._tokenizer = None
        if tokenizer is not None:
            from .tokenization import TokenizerWrapper
            self._tokenizer = tokenizer if isinstance(tokenizer, TokenizerWrapper) else \
                TokenizerWrapper(tokenizer, max_length=getattr(self.config.tokenizer, "max_length", 2048))
        self._engine = None
        self._memory: dict[str, Sequence[Mapping[str, Any]]] = {}
        self.introspector = DatasetIntrospector(self.token)

    @classmethod
    @reference_kwargs(config_path="path_or_dict")
    def from_config(cls, path_or_dict, token: str | None = None, trust_remote_code: bool = False) -> Result:
        r = load_config_dict(path_or_dict) if isinstance(path_or_dict, Mapping) else load_config(path_or_dict)
        if r.is_err():
            return r
        return Ok(cls(r.unwrap(), token, trust_remote_code))

    # ---------------------------------------------------------------- lazy parts
    @property
    def tokenizer(self):
        return self._ensure_tokenizer()

    def _ensure_tokenizer(self):
        if self._tokenizer is None:
            self._tokenizer = create_tokenizer(self.config.tokenizer, token=self.token,
                                               trust_remote_code=self.trust_remote_code)
        return self._tokenizer

    def _ensure_prompt_engine(self) -> PromptEngine:
        if self._engine is None:
            tok = self._ensure_tokenizer()
            pe = self.config.prompt_engine
            max_len = pe.max_length if pe is not None else self.config.tokenizer.max_length
            cd = self.config.preprocessing.content_distribution
            dist = None
            if cd.enabled or pe is None or TrainingStage(pe.stage) == TrainingStage.FINE_TUNING:
                dist = TokenAwareContentDistributor(cd.mode if cd.enabled else ContentDistributionMode.PROPORTIONAL,
                                                    max_len, special_tokens_budget=cd.special_tokens_budget, tokenizer=tok)
            if pe is not None:
                self._engine = PromptEngine.from_config(pe, tok, dist, self.config.prompt)
            else:
                self._engine = PromptEngine.from_legacy(self.config.prompt, tok, max_len, dist)
        return self._engine

    # ---------------------------------------------------------------- datasets
    def register_dataset(self, split: str, rows: Sequence[Mapping[str, Any]]) -> None:
        self._memory[split] = rows

    def discover(self) -> Result:
        if self._memory:
            return self.introspector.discover(self._memory)
        ds = self.config.dataset
        return self.introspector.discover(ds.path or ds.name, ds.config_name)

    def get_splits(self) -> list[str]:
        ds = self.config.dataset
        if ds.splits:
            return list(ds.splits)
        if self._memory:
            return list(self._memory)
        md = self.discover()
        return list(md.unwrap().splits) if md.is_ok() else []

    def get_stage_splits(self, stage: str) -> list[str]:
        """Split names of one curriculum stage; empty for an unknown stage or a dataset without stages."""
        st = self.config.dataset.stages.get(stage) if self.config.dataset.stages else None
        return list(st.splits) if st is not None else []

    def load_dataset(self, split: str = "train", streaming: bool | None = None) -> Result:
        """`streaming`: override the dataset's configured mode for this call (hub datasets only; local files and
        registered rows are always materialised)."""
        if streaming is not None and streaming != self.config.dataset.streaming:
            import dataclasses
            saved = self.config
            self.config = dataclasses.replace(saved, dataset=dataclasses.replace(saved.dataset, streaming=bool(streaming)))
            try:
                return self.load_dataset(split)
            finally:
                self.config = saved
        ds = self.config.dataset
        spec = ds.splits.get(split)
        real = spec.name if spec is not None else split
        try:
            rows = self._load_rows(real, split)
        except PipelineError as e:
            return Err(e)
        if spec is not None:
            if spec.shuffle and hasattr(rows, "__len__"):
                import random
                idx = list(range(len(rows)))
                random.Random(spec.seed).shuffle(idx)
                rows = [rows[i] for i in idx]
            if spec.sample_size is not None and hasattr(rows, "__len__"):
                rows = rows[:spec.sample_size] if isinstance(rows, list) else rows.select(range(min(spec.sample_size, len(rows))))
        return Ok(rows)

    def _load_rows(self, real: str, alias: str):
        ds = self.config.dataset
        for k in (alias, real):
            if k in self._memory:
                return self._memory[k]
        src = ds.path or ds.name
        if str(src).lower() == "synthetic":
            from .synthetic import SyntheticTokenDataset
            raise DataLoadingError("the synthetic dataset is token-level: use synthetic_dataloader(...) directly")
        p = Path(str(src))
        if p.exists():
            from .local_datasets import load_local_dataset
            if p.is_file():
                return load_local_dataset(p)
            for ext in (".jsonl", ".json", ".parquet", ".csv", ".txt"):
                if (p / f"{real}{ext}").exists():
                    return load_local_dataset(p / f"{real}{ext}")
            raise SplitNotFoundError(f"split {real!r} not found under {p}")
        try:
            import datasets
            return datasets.load_dataset(ds.name, ds.config_name, split=real, streaming=ds.streaming,
                                         revision=ds.revision, token=self.token, trust_remote_code=self.trust_remote_code)
        except Exception as e:   # noqa: BLE001
            raise DatasetNotFoundError(f"cannot load dataset {ds.name!r} split {real!r}", cause=e)

    def get_preprocessed_dataset(self, split: str = "train", rank: int = 0, world_size: int = 1,
                                 streaming: bool | None = None) -> Result:
        r = self.load_dataset(split, streaming)
        if r.is_err():
            return r
        try:
            engine = self._ensure_prompt_engine()
        except PipelineError as e:
            return Err(e)
        ds = self.config.dataset
        return Ok(create_preprocessed_dataset(r.unwrap(), engine, streaming=ds.streaming if streaming is None else streaming,
                                              column_mapping=dict(ds.column_mapping), rank=rank, world_size=world_size))

    def get_dataloader(self, split: str = "train", batch_size: int | None = None, distributed: bool = False,
                       rank: int = 0, world_size: int = 1, shuffle: bool | None = None,
                       num_workers: int | None = None) -> Result:
        r = self.get_preprocessed_dataset(split, rank, world_size)
        if r.is_err():
            return r
        dl = self.config.dataloader
        tok = self._ensure_tokenizer()
        collate = create_collate_fn(tok.pad_token_id, padding_side=self.config.tokenizer.padding_side,
                                    output_schema=self.config.output_schema)
        try:
            return Ok(build_dataloader(
                r.unwrap(), batch_size=batch_size or dl.batch_size,
                shuffle=(dl.shuffle if shuffle is None else shuffle) and split.startswith("train"), seed=dl.seed,
                num_workers=dl.num_workers if num_workers is None else num_workers, pin_memory=dl.pin_memory, drop_last=dl.drop_last, collate_fn=collate,
                distributed=distributed, rank=rank, world_size=world_size, prefetch_factor=dl.prefetch_factor,
                persistent_workers=dl.persistent_workers))
        except PipelineError as e:
            return Err(e)


def create_pipeline(path_or_dict, **kw) -> DataPipeline:
    return DataPipeline.from_config(path_or_dict, **kw).unwrap()
