"""Compiles the CUDA sources beside this file for sm_100a and loads them with ctypes.

Each source becomes one shared library under ``csrc/_build/`` (or
``$DLI_B200_BUILD_DIR``), named after the source, its preprocessor defines and a
hash of everything that went into it, so a stale build is never loaded.  A
library is compiled at its first use; only what a model needs is built.  While
``nvcc`` runs, a line is printed now and then so a first call does not look hung.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

SRC_DIR = Path(__file__).resolve().parent
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class ExtensionError(RuntimeError):
    """The CUDA extension could not be built or loaded; there is no fallback."""


def _say(msg: str) -> None:
    print(f"[dli_b200] {msg}", file=sys.stderr, flush=True)


_build_dir: Path | None = None


def build_dir() -> Path:
    """Where the libraries go: decided once per process (several threads may ask at the same time)."""
    global _build_dir
    with _lock:
        if _build_dir is None:
            env = os.environ.get("DLI_B200_BUILD_DIR")
            cand = Path(env) if env else SRC_DIR / "_build"
            try:
                cand.mkdir(parents=True, exist_ok=True)
                probe = cand / f".w{os.getpid()}_{threading.get_ident()}"
                probe.write_text("")
                probe.unlink()
                _build_dir = cand
            except OSError:
                fallback = Path(tempfile.gettempdir()) / f"dli_b200_build_{os.getuid()}"
                fallback.mkdir(parents=True, exist_ok=True)
                _build_dir = fallback
        return _build_dir


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise ExtensionError("nvcc not found (set NVCC or put it on PATH): the engine's kernels cannot be built")


def _digest(source: str, defines: dict[str, object]) -> str:
    h = hashlib.sha256()
    for path in [SRC_DIR / source, *sorted(SRC_DIR.glob("*.cuh")), *sorted(SRC_DIR.glob("*.h"))]:  # every header a source may include
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def library_path(source: str, defines: dict[str, object] | None = None) -> Path:
    defines = defines or {}
    tag = "".join(f"_{k.lower()}{v}" for k, v in sorted(defines.items()))
    return build_dir() / f"dli_{Path(source).stem}{tag}_{_digest(source, defines)}.so"


def compile_library(source: str, defines: dict[str, object] | None = None, extra: list[str] | None = None) -> Path:
    """Compile one source if its library is not there yet; returns the library's path."""
    defines = defines or {}
    out = library_path(source, defines)
    if out.exists():
        return out
    cmd = [_nvcc(), *NVCC_FLAGS, *(extra or []), *[f"-D{k}={v}" for k, v in sorted(defines.items())]]
    tmp = out.with_suffix(f".tmp{os.getpid()}_{threading.get_ident()}.so")
    cmd += ["-o", str(tmp), str(SRC_DIR / source)]
    _say(f"compiling {out.name} (first use) ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            log, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            _say(f"  still compiling {out.name}: {time.time() - t0:.0f} s")
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise ExtensionError(f"nvcc failed for {source}:\n{log}")
    os.replace(tmp, out)  # atomic: a concurrent process sees the whole file or none
    _say(f"built {out.name} in {time.time() - t0:.1f} s")
    for old in out.parent.glob(out.name[: -len("0123456789abcdef.so")] + "*.so"):  # libraries of earlier versions of this source
        if old != out and len(old.name) == len(out.name) and ".tmp" not in old.name:
            try:
                old.unlink()  # a process that has one loaded keeps its mapping
            except OSError:
                pass
    return out


def load_library(source: str, defines: dict[str, object] | None = None, extra: list[str] | None = None) -> ctypes.CDLL:
    key = f"{source}|{sorted((defines or {}).items())}"  # sources are hashed once per process, not per call
    with _lock:
        lib = _loaded.get(key)
    if lib is not None:
        return lib
    path = compile_library(source, defines, extra)
    try:
        lib = ctypes.CDLL(str(path))
    except OSError as exc:
        raise ExtensionError(f"cannot load {path}: {exc}") from exc
    with _lock:
        _loaded[key] = lib
    return lib


def compile_many(jobs: list[tuple[str, dict[str, object] | None]]) -> list[Path]:
    """Compile several libraries side by side (used at model build and by the build check)."""
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        return list(pool.map(lambda j: compile_library(j[0], j[1]), jobs))
