"""Keyword compatibility with the reference's function signatures.

Many functions here have a counterpart of the same name in the reference whose parameters are spelled differently
(`input_` for `x`, `process_group` for `group`, ...) or which takes options that have no effect in this framework
(`async_op`, `inplace`, `use_triton`).  `reference_kwargs` lets a function take both spellings without changing its
own signature: renamed keywords are passed on under this framework's name; accepted-only options are dropped when they
carry a neutral value and refused (NotImplementedError) when they ask for something that is not done here, so that no
request is ignored silently.
"""
from __future__ import annotations

import functools
import inspect

ANY = object()          # marks an accepted option whose value never matters here
NEUTRAL = (None, False, 0, 0.0, "", "none", "auto")


def reference_kwargs(_accept: dict | tuple | None = None, **renames: str):
    """`@reference_kwargs(input_="x", process_group="group")` and / or `@reference_kwargs({"async_op": (False,)})`.

    `_accept` maps an option name to the tuple of values that are fine to drop (or ANY); a tuple / list of names accepts
    each with the usual neutral values (None, False, 0, "", "none", "auto")."""
    accept = {n: NEUTRAL for n in _accept} if isinstance(_accept, (tuple, list)) else dict(_accept or {})

    def deco(fn):
        sig = inspect.signature(fn)

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            for ref, ours in renames.items():
                if ref in kwargs:
                    if ours in kwargs:
                        raise TypeError(f"{fn.__name__}() got both {ref!r} and {ours!r}")
                    kwargs[ours] = kwargs.pop(ref)
            for name, neutral in accept.items():
                if name in kwargs:
                    v = kwargs.pop(name)
                    if neutral is not ANY and not any(v is n or (type(v) is type(n) and v == n) for n in neutral):
                        raise NotImplementedError(f"{fn.__name__}(): {name}={v!r} is not supported by this framework")
            return fn(*args, **kwargs)

        params = list(sig.parameters.values())
        tail = [p for p in params if p.kind is inspect.Parameter.VAR_KEYWORD]
        head = [p for p in params if p.kind is not inspect.Parameter.VAR_KEYWORD]
        extra = [inspect.Parameter(n, inspect.Parameter.KEYWORD_ONLY, default=None)
                 for n in list(renames) + list(accept) if n not in sig.parameters]
        wrapper.__signature__ = sig.replace(parameters=head + extra + tail)
        wrapper.__reference_renames__ = {**getattr(fn, "__reference_renames__", {}), **renames}
        return wrapper

    return deco
