"""Builds the sm_100a kernel libraries with nvcc and loads them with ctypes.

Each ``csrc/<name>.cu`` becomes one shared library ``_build/lib<name>-<hash>.so`` that exports
plain C functions.  A library is compiled the first time one of its functions is asked for (so a
run compiles only what its model and precision need) and is reused afterwards; the hash covers
the source, the shared headers, the flags and the compiler version, so an edited source never
meets a stale binary.  There is no fallback: a missing compiler or a failed build raises
``KernelBuildError``.
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
from pathlib import Path

CSRC_DIR = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC"]


class KernelBuildError(RuntimeError):
    """The CUDA kernels could not be compiled or loaded; the engine cannot run without them."""


_lock = threading.Lock()
_dir_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def _log(msg: str) -> None:
    print(f"[gpullama3.java_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("NVCC"), shutil.which("nvcc")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            candidates.append(os.path.join(home, "bin", "nvcc"))
    for c in candidates:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH, $CUDA_HOME, /usr/local/cuda); "
                           "the engine has no path without its CUDA kernels")


_nvcc_version_cache: list[str] = []


def _nvcc_version(nvcc: str) -> str:
    if not _nvcc_version_cache:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
        _nvcc_version_cache.append(out.strip().splitlines()[-1] if out.strip() else "unknown")
    return _nvcc_version_cache[0]


def available_libraries() -> list[str]:
    return sorted(p.stem for p in CSRC_DIR.glob("*.cu"))


def _source_hash(name: str, nvcc: str) -> str:
    h = hashlib.sha256()
    h.update((CSRC_DIR / f"{name}.cu").read_bytes())
    for header in sorted(list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.h"))):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    h.update(_nvcc_version(nvcc).encode())
    return h.hexdigest()[:12]


_build_dir_cache: list[Path] = []


def build_dir() -> Path:
    """The in-tree ``_build`` folder when it can be written, else a per-user temporary folder."""
    if not _build_dir_cache:
        with _dir_lock:
            if not _build_dir_cache:
                _build_dir_cache.append(_find_build_dir())
    return _build_dir_cache[0]


def _find_build_dir() -> Path:
    override = os.environ.get("GPULLAMA3_B200_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC_DIR.parent / "_build"
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".write-probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"gpullama3_java_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def library_path(name: str) -> Path:
    nvcc = find_nvcc()
    return build_dir() / f"lib{name}-{_source_hash(name, nvcc)}.so"


def compile_library(name: str, *, verbose_ptxas: bool = False) -> Path:
    """Compile ``csrc/<name>.cu`` if its library is not there yet; returns the library's path."""
    src = CSRC_DIR / f"{name}.cu"
    if not src.is_file():
        raise KernelBuildError(f"no kernel source {src}")
    nvcc = find_nvcc()
    out = build_dir() / f"lib{name}-{_source_hash(name, nvcc)}.so"
    if out.is_file():
        return out
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC_DIR), "-o", str(tmp), str(src)]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    _log(f"compiling {src.name} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _log(f"  still compiling {src.name} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        output, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {src.name} (exit {proc.returncode}):\n{output}")
    os.replace(tmp, out)
    _log(f"compiled {src.name} in {time.time() - t0:.1f} s")
    if verbose_ptxas:
        print(output, file=sys.stderr)
    # drop older builds of the same source
    for old in out.parent.glob(f"lib{name}-*.so"):
        if old != out and ".tmp" not in old.name:
            try:
                old.unlink()
            except OSError:
                pass
    return out


def library(name: str) -> ctypes.CDLL:
    """The loaded kernel library ``name``, compiled first if needed."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
    return lib


def build_all(names: list[str] | None = None, jobs: int | None = None) -> list[Path]:
    """Compile every kernel library (or ``names``) in parallel.  Needs no GPU."""
    from concurrent.futures import ThreadPoolExecutor

    names = names or available_libraries()
    jobs = jobs or min(len(names), os.cpu_count() or 1)
    with ThreadPoolExecutor(max_workers=max(1, jobs)) as pool:
        return list(pool.map(compile_library, names))
