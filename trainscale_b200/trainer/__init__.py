"""Trainers.  `SOTATrainer` (YAML-driven) lives in `sota_trainer`, the `Trainer` family in `base`.

The aliases below are the names under which data_pipeline/trainer/__init__.py re-exports parts of its configuration
module; they are resolved on first use so that importing this package stays cheap.
"""
from __future__ import annotations

import importlib

_ALIASES = {
    "SOTATrainingMode": ("..config.sota_config", "TrainingMode"),
    "SOTAPrecision": ("..config.sota_config", "Precision"),
    "SOTAOptimizerType": ("..config.sota_config", "OptimizerType"),
    "SOTASchedulerType": ("..config.sota_config", "SchedulerType"),
    "SOTALossType": ("..config.sota_config", "LossType"),
    "SOTADeviceType": ("..config.sota_config", "DeviceType"),
    "SOTAQuantizationConfig": ("..config.sota_config", "QuantizationConfig"),
    "SOTATrainingState": (".sota_trainer", "TrainingState"),
    "SOTAConfig": ("..config.sota_config", "SOTAConfig"),
    "SOTATrainer": (".sota_trainer", "SOTATrainer"),
    "create_trainer": (".sota_trainer", "create_trainer"),
    "Trainer": (".base", "Trainer"),
}


def __getattr__(name: str):
    if name in _ALIASES:
        module, attr = _ALIASES[name]
        value = getattr(importlib.import_module(module, __name__), attr)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_ALIASES))
