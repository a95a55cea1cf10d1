"""Process-wide switch for activation recomputation, consulted where layers are wrapped in a checkpoint.

`override()` is None (each module decides as configured), False (inside `no_checkpoint()`: run every layer plainly)
or True (inside `force_checkpoint()`: recompute wherever a layer is configured for it, even outside training mode, as
long as gradients are being recorded).
"""
from __future__ import annotations

import contextlib

_STATE: list = [None]


def override():
    return _STATE[0]


def wanted(configured: bool, training: bool) -> bool:
    """Whether a layer that is `configured` for recomputation should be checkpointed now."""
    if _STATE[0] is False or not configured:
        return False
    return training or _STATE[0] is True


@contextlib.contextmanager
def scoped(value):
    prev = _STATE[0]
    _STATE[0] = value
    try:
        yield
    finally:
        _STATE[0] = prev
