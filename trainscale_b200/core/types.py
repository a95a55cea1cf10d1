"""Result type used by the data half of the API (`DataPipeline.from_config(...) -> Result`).

Same surface as data_pipeline/core/types.py:27-240 (Ok / Err / is_ok / unwrap / map_result / flat_map /
map_err), written as two small frozen dataclasses with methods, plus the free functions.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Generic, TypeVar, Union

T = TypeVar("T")
U = TypeVar("U")
E = TypeVar("E")
F = TypeVar("F")


@dataclass(frozen=True)
class Ok(Generic[T]):
    value: T

    def is_ok(self) -> bool:
        return True

    def is_err(self) -> bool:
        return False

    def unwrap(self) -> T:
        return self.value

    def unwrap_or(self, default):
        return self.value

    def map(self, fn):
        return Ok(fn(self.value))

    def and_then(self, fn):
        return fn(self.value)

    def __repr__(self):
        return f"Ok({self.value!r})"


@dataclass(frozen=True)
class Err(Generic[E]):
    error: E

    def is_ok(self) -> bool:
        return False

    def is_err(self) -> bool:
        return True

    def unwrap(self):
        if isinstance(self.error, BaseException):
            raise self.error
        raise ValueError(f"called unwrap on Err: {self.error!r}")

    def unwrap_or(self, default):
        return default

    def map(self, fn):
        return self

    def and_then(self, fn):
        return self

    def __repr__(self):
        return f"Err({self.error!r})"


Result = Union[Ok[T], Err[E]]


def is_ok(r) -> bool:
    return isinstance(r, Ok)


def is_err(r) -> bool:
    return isinstance(r, Err)


def unwrap(r):
    return r.unwrap()


def unwrap_err(r):
    if isinstance(r, Err):
        return r.error
    raise ValueError(f"called unwrap_err on Ok: {r.value!r}")


def unwrap_or(r, default):
    return r.value if isinstance(r, Ok) else default


def unwrap_or_else(r, fn: Callable):
    return r.value if isinstance(r, Ok) else fn(r.error)


def map_result(r, fn: Callable):
    return Ok(fn(r.value)) if isinstance(r, Ok) else r


def flat_map(r, fn: Callable):
    return fn(r.value) if isinstance(r, Ok) else r


def map_err(r, fn: Callable):
    return Err(fn(r.error)) if isinstance(r, Err) else r
