"""Compiles the CUDA sources under csrc/ for sm_100a with nvcc and loads them with ctypes.

Each source file becomes one shared library under `<package>/_build/` (or, when that folder
cannot be written, under a per-user folder in the system's temporary directory).  A library is
named after its source, its `-D` specialisation and a hash of everything that went into it, so
a changed source or flag is rebuilt and an unchanged one is loaded as it is.  The sources use
only the CUDA runtime (no torch headers), so a file compiles in seconds; what a model needs is
compiled at its first use, with a progress line on stderr for every file.

There is no fallback: if nvcc is missing or a compile fails, `KernelBuildError` is raised.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import pathlib
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, Optional, Sequence

from ..errors import KernelBuildError

CSRC = pathlib.Path(__file__).resolve().parent.parent / "csrc"
_PACKAGE_BUILD = pathlib.Path(__file__).resolve().parent.parent / "_build"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
              "--expt-relaxed-constexpr", "--extended-lambda"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise KernelBuildError("nvcc not found: the engine's kernels cannot be built (set NVCC or put "
                           "nvcc on PATH); there is no fallback path")


_build_dir: Optional[pathlib.Path] = None


def build_dir() -> pathlib.Path:
    """The folder libraries are written to: in-tree when writable, else per-user temporary."""
    global _build_dir
    if _build_dir is None:
        _build_dir = _pick_build_dir()
    return _build_dir


def _pick_build_dir() -> pathlib.Path:
    override = os.environ.get("BARE_CUDA_B200_BUILD_DIR")
    candidates = [pathlib.Path(override)] if override else []
    candidates.append(_PACKAGE_BUILD)
    candidates.append(pathlib.Path(tempfile.gettempdir()) / f"bare_cuda_4gib_b200-build-{os.getuid()}")
    for c in candidates:
        try:
            c.mkdir(parents=True, exist_ok=True)
            probe = c / f".writable-{os.getpid()}-{threading.get_ident()}"
            probe.write_text("")
            probe.unlink()
            return c
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {[str(c) for c in candidates]}")


def _source_hash(source: pathlib.Path, defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    h.update(source.read_bytes())
    for header in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + list(defines)).encode())
    return h.hexdigest()[:16]


def library_path(source_name: str, defines: Sequence[str] = ()) -> pathlib.Path:
    source = CSRC / source_name
    tag = "".join(c if c.isalnum() else "_" for c in "_".join(d.lstrip("-D") for d in defines))
    stem = source.stem + (f"-{tag}" if tag else "")
    return pathlib.Path(f"{stem}-{_source_hash(source, defines)}.so")


def _find_built(name: pathlib.Path) -> Optional[pathlib.Path]:
    for folder in (_PACKAGE_BUILD, build_dir()):
        p = folder / name
        if p.exists():
            return p
    return None


def compile_library(source_name: str, defines: Sequence[str] = (), verbose: bool = True) -> pathlib.Path:
    """Builds (if needed) and returns the shared library for one source and specialisation."""
    name = library_path(source_name, defines)
    found = _find_built(name)
    if found is not None:
        return found
    out_dir = build_dir()
    target = out_dir / name
    tmp = out_dir / f".{name}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *defines, "-I", str(CSRC), str(CSRC / source_name),
           "-o", str(tmp)]
    if verbose:
        print(f"[bare_cuda_4gib_b200] compiling {source_name} {' '.join(defines)} for sm_100a ...",
              file=sys.stderr, flush=True)
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[bare_cuda_4gib_b200]   ... still compiling {source_name} "
                      f"({time.time() - start:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {source_name} {list(defines)}:\n{output}")
    os.replace(tmp, target)
    if verbose:
        print(f"[bare_cuda_4gib_b200]   built {target.name} in {time.time() - start:.1f} s",
              file=sys.stderr, flush=True)
    return target


def load_library(source_name: str, defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = str(library_path(source_name, defines))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(source_name, defines)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[key] = lib
        return lib


def compile_many(jobs: Iterable[tuple], verbose: bool = True) -> None:
    """Compiles several (source, defines) pairs in parallel threads (nvcc runs as subprocesses)."""
    jobs = [j for j in jobs if _find_built(library_path(*j)) is None]
    errors = []

    def work(job):
        try:
            compile_library(*job, verbose=verbose)
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
