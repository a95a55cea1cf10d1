"""ctypes loader for the in-tree CUDA libraries.

A library is loaded on first use.  On a machine with a GPU a missing library is an error (the CUDA
path must be the one that runs); on a CPU-only machine the callers use their PyTorch reference math.
"""
from __future__ import annotations

import ctypes
import functools

import torch

from .build import build_all, lib_path

_ERR_NAMES = {0: "none", 1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad argument", 4: "tmem",
              5: "access outside its tensor (debug build: skipped)"}


class KernelError(RuntimeError):
    pass


def cuda_available() -> bool:
    return torch.cuda.is_available()


@functools.lru_cache(maxsize=None)
def load(name: str) -> ctypes.CDLL:
    path = lib_path(name)
    if not path.exists():
        build_all()
    if not path.exists():
        raise KernelError(f"CUDA library {path} is missing; run `python -m trainscale_b200.ops.build`")
    return ctypes.CDLL(str(path))


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    """Device address of `t` for a kernel argument.  The kernels launch on the CURRENT device's stream, so a tensor
    that lives on another GPU is refused here, on the host, instead of faulting on the device."""
    if t is None:
        return ctypes.c_void_p(0)
    if t.is_cuda and t.device.index != torch.cuda.current_device():
        raise KernelError(f"tensor on {t.device} passed to a kernel while the current device is "
                          f"cuda:{torch.cuda.current_device()}; call torch.cuda.set_device (or use torch.cuda.device) first")
    return ctypes.c_void_p(t.data_ptr())


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def device_error(name: str) -> tuple[int, int, int, int]:
    """Read (and leave untouched) the error word of library `name`: (code, site, block, extra)."""
    lib = load(name)
    buf = (ctypes.c_uint * 4)()
    getattr(lib, f"ts_{name}_get_error")(buf)
    return tuple(int(x) for x in buf)


def clear_device_error(name: str) -> None:
    getattr(load(name), f"ts_{name}_clear_error")()


def raise_on_device_error(name: str) -> None:
    code, site, block, extra = device_error(name)
    if code:
        clear_device_error(name)
        raise KernelError(f"{name} kernel reported '{_ERR_NAMES.get(code, code)}' at site {site} "
                          f"(block {block}, extra {extra})")


# number of launcher calls made through `check` (each is at least one kernel of this library)
LAUNCHES = 0
_orig_check = check


def check(rc: int, what: str) -> None:  # noqa: F811
    global LAUNCHES
    LAUNCHES += 1
    _orig_check(rc, what)


def raise_on_any_device_error() -> None:
    """Check the error word of every library that has been built."""
    from .build import sources
    for src in sources():
        if lib_path(src.stem).exists():
            raise_on_device_error(src.stem)
