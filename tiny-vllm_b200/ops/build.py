"""Compile the CUDA sources for sm_100a and load them.

Each ``csrc/<name>.cu`` becomes one shared library that is compiled with nvcc at
its first use and loaded with ctypes; its ``extern "C"`` launchers take raw
device pointers and a stream.  Libraries are kept beside the sources in
``csrc/_build`` (or, if that folder cannot be written, in a per-user folder
under the system's temporary directory), named by a hash of the source, the
headers and the flags, so an edited source is rebuilt and an unchanged one is
not.  A model triggers only the libraries its parts call.

There is no fallback: if nvcc is absent or a source does not compile, the
call raises :class:`KernelBuildError`.  The reference builds its three sources
with torch's JIT extension loader (tinyvllm/kernels/_extension.py:10-42).
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
)
# libraries and the other linker inputs some sources need
EXTRA_LINK: dict[str, tuple[str, ...]] = {}

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    """A CUDA source could not be compiled or loaded."""


def source_names() -> tuple[str, ...]:
    return tuple(sorted(path.stem for path in CSRC.glob("*.cu")))


def _find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise KernelBuildError(
        "nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
        "the CUDA kernels cannot be built and there is no other path")


_INCLUDE = re.compile(r'^\s*#\s*include\s*"([^"]+)"', re.MULTILINE)


def _sources_of(name: str) -> list[Path]:
    """``csrc/<name>.cu`` and the files of this folder that it includes, directly or not."""
    found: dict[str, Path] = {}
    waiting = [CSRC / f"{name}.cu"]
    while waiting:
        path = waiting.pop()
        if path.name in found or not path.is_file():
            continue
        found[path.name] = path
        waiting.extend(CSRC / included for included in _INCLUDE.findall(path.read_text(errors="replace")))
    return [found[key] for key in sorted(found)]


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + EXTRA_LINK.get(name, ())).encode())
    for path in _sources_of(name):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()[:16]


def _build_dirs() -> list[Path]:
    return [CSRC / "_build",
            Path(tempfile.gettempdir()) / f"tinyvllm_b200_build_{os.getuid()}"]


def _usable_dir() -> Path:
    for folder in _build_dirs():
        try:
            folder.mkdir(parents=True, exist_ok=True)
            with tempfile.NamedTemporaryFile(dir=folder, prefix=".probe_"):
                pass
            return folder
        except OSError:
            continue
    raise KernelBuildError("no writable folder for the compiled kernels: " +
                           ", ".join(str(p) for p in _build_dirs()))


def library_path(name: str) -> Path | None:
    """Path of the up-to-date library of ``name`` if it has been built."""
    filename = f"tvb200_{name}_{_digest(name)}.so"
    for folder in _build_dirs():
        if (folder / filename).is_file():
            return folder / filename
    return None


def compile_library(name: str, *, verbose: bool = True) -> Path:
    """Compile ``csrc/<name>.cu`` unless its library is already there."""
    source = CSRC / f"{name}.cu"
    if not source.is_file():
        raise KernelBuildError(f"no CUDA source named {name!r} in {CSRC}")
    existing = library_path(name)
    if existing is not None:
        return existing
    nvcc = _find_nvcc()
    folder = _usable_dir()
    target = folder / f"tvb200_{name}_{_digest(name)}.so"
    partial = folder / f".{target.name}.{os.getpid()}.{threading.get_ident()}.tmp"
    command = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-o", str(partial), str(source),
               *EXTRA_LINK.get(name, ())]
    if verbose:
        print(f"[tinyvllm_b200] compiling {source.name} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = process.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[tinyvllm_b200]   still compiling {source.name} "
                      f"({time.time() - started:.0f} s)", file=sys.stderr, flush=True)
    if process.returncode != 0:
        partial.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed on {source.name}:\n{output}")
    os.replace(partial, target)
    for stale in folder.glob(f"tvb200_{name}_*.so"):       # builds of older versions of this source
        if stale != target:
            stale.unlink(missing_ok=True)
    if verbose:
        print(f"[tinyvllm_b200] built {target.name} in {time.time() - started:.1f} s",
              file=sys.stderr, flush=True)
    return target


def compile_all(*, verbose: bool = True, jobs: int = 4) -> list[Path]:
    """Compile every source (several at a time); used by the build check."""
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=jobs) as pool:
        return list(pool.map(lambda n: compile_library(n, verbose=verbose), source_names()))


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library of ``csrc/<name>.cu``, compiled first if need be."""
    with _lock:
        library = _loaded.get(name)
        if library is None:
            path = compile_library(name)
            try:
                library = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelBuildError(f"cannot load {path}: {exc}") from exc
            _loaded[name] = library
        return library
