"""trainscale_b200: YAML-driven LLM training and inference on NVIDIA B200 (sm_100a).

Public surface (mirrors the reference package's flat namespace, data_pipeline/trainer/__init__.py:15-319):
configuration (`SOTAConfig`, `load_config`), data (`DataPipeline`, `PromptEngine`, `TokenizerWrapper`, collate /
DataLoader builders), model (`LlamaForCausalLM`, `build_model`), training (`SOTATrainer`, `create_trainer`,
`FlatShardedEngine`), losses / optimizers / schedulers factories, inference (`SOTAInferenceEngine`).
"""
__version__ = "0.1.0"

_LAZY = {
    "SOTAConfig": "trainscale_b200.config.sota_config", "load_config": "trainscale_b200.config.data_schema",
    "PipelineConfig": "trainscale_b200.config.data_schema", "DataPipeline": "trainscale_b200.data.pipeline",
    "create_pipeline": "trainscale_b200.data.pipeline", "PromptEngine": "trainscale_b200.data.prompt_engine",
    "TokenizerWrapper": "trainscale_b200.data.tokenization", "create_tokenizer": "trainscale_b200.data.tokenization",
    "create_collate_fn": "trainscale_b200.data.collate", "build_dataloader": "trainscale_b200.data.dataloader_factory",
    "LlamaConfig": "trainscale_b200.models.llama", "LlamaForCausalLM": "trainscale_b200.models.llama",
    "build_model": "trainscale_b200.models.llama", "SOTATrainer": "trainscale_b200.trainer.sota_trainer",
    "create_trainer": "trainscale_b200.trainer.sota_trainer", "Trainer": "trainscale_b200.trainer.base",
    "FlatShardedEngine": "trainscale_b200.parallel.flat_engine", "EngineConfig": "trainscale_b200.parallel.flat_engine",
    "create_loss": "trainscale_b200.losses", "LossRegistry": "trainscale_b200.losses",
    "create_optimizer": "trainscale_b200.optim", "create_scheduler": "trainscale_b200.schedulers",
    "SOTAInferenceEngine": "trainscale_b200.inference", "SOTAAsyncStreamEngine": "trainscale_b200.inference",
    "GenerationParams": "trainscale_b200.inference", "CallbackHandler": "trainscale_b200.callbacks",
    "Ok": "trainscale_b200.core.types", "Err": "trainscale_b200.core.types", "PreferenceTrainer": "trainscale_b200.rl",
    "KernelPatcher": "trainscale_b200.registry", "export_model": "trainscale_b200.export",
}


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'trainscale_b200' has no attribute {name!r}")
    import importlib
    return getattr(importlib.import_module(mod), name)


__all__ = sorted(_LAZY)
