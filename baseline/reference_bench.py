"""Reference arm of bench.py: runs the unmodified reference (installed under baseline/_ref) on the same metric."""
from __future__ import annotations

import json
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"


def run_reference(args) -> dict:
    if not (REF_DIR / "data_pipeline").exists():
        return {"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"}
    from .reference_runner import run
    return run(args)
