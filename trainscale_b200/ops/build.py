"""In-tree build of the sm_100a CUDA libraries.

Each ``csrc/<name>.cu`` becomes ``lib/libts_<name>.so`` (plain ``extern "C"`` entry points, loaded with
ctypes, no torch headers, so a full rebuild takes seconds).  ``nvcc`` cross-compiles without a GPU.

Debug build: ``TS_DEBUG=1`` selects ``lib_debug/`` (built with ``-DTS_DEBUG=1``): every GEMM epilogue store and every
peer read of the fused reduce-scatter is checked against the extent of its tensor, an access outside it is skipped and
recorded in the library's error word (`ops/_lib.raise_on_any_device_error`), and `parallel.symm.SymmetricHeap` puts
canary words around every symmetric buffer.  Slower; for chasing an indexing bug or a suspected overrun.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent.parent
CSRC_DIR = PKG_DIR / "csrc"
DEBUG = os.environ.get("TS_DEBUG", "0") == "1"
LIB_DIR = PKG_DIR / ("lib_debug" if DEBUG else "lib")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--shared", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    p = Path("/usr/local/cuda/bin/nvcc")
    return str(p) if p.exists() else None


def sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def lib_path(name: str) -> Path:
    return LIB_DIR / f"libts_{name}.so"


def _stale(src: Path, out: Path) -> bool:
    if not out.exists():
        return True
    newest = max([src.stat().st_mtime] + [h.stat().st_mtime for h in CSRC_DIR.glob("*.cuh")] +
                 [h.stat().st_mtime for h in CSRC_DIR.glob("*.h")])
    return out.stat().st_mtime < newest


def build_all(force: bool = False, verbose: bool = False, debug: bool | None = None) -> list[Path]:
    """Compile every stale library; returns the list of library paths. Raises on a compile error.
    `debug`: build the checked variant into lib_debug/ (default: what TS_DEBUG selected for this process)."""
    nvcc = find_nvcc()
    debug = DEBUG if debug is None else debug
    lib_dir = PKG_DIR / ("lib_debug" if debug else "lib")
    lib_dir.mkdir(exist_ok=True)
    outs = []
    procs = []
    for src in sources():
        out = lib_dir / f"libts_{src.stem}.so"
        outs.append(out)
        if not force and not _stale(src, out):
            continue
        if nvcc is None:
            raise RuntimeError(f"nvcc not found and {out.name} is missing or stale")
        cmd = [nvcc, *NVCC_FLAGS, *(["-DTS_DEBUG=1"] if debug else []), "-o", str(out), str(src)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), file=sys.stderr)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        log, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{log}")
        if verbose and log:
            print(log, file=sys.stderr)
    return outs


if __name__ == "__main__":
    for o in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print(o)
