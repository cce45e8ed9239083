"""Compiles the CUDA sources under csrc/ for sm_100a and loads them with ctypes.

The mechanism is fastllm-py's: nvcc -> shared object -> `ctypes.CDLL`
(native/build.sh, fastllm_py/kernels/marlin.py:56-95), but the build is driven
from Python so that a fresh checkout compiles what it needs at the first call:
each library is one .cu file plus the `-D` defines it was asked for (a head
size, say), named by a hash of its sources and flags, built once and reused.

There is no fallback: a library that cannot be built or loaded raises.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden"]

_loaded: dict = {}
_lock = threading.RLock()


class NativeBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    exe = os.environ.get("NVCC") or shutil.which("nvcc")
    if exe is None and Path("/usr/local/cuda/bin/nvcc").exists():
        exe = "/usr/local/cuda/bin/nvcc"
    if exe is None:
        raise NativeBuildError(
            "nvcc not found: the engine's CUDA kernels must be compiled for sm_100a and "
            "there is no other way to run it (set NVCC or put nvcc on PATH)")
    return exe


_build_dir_cache = None


def _build_dir() -> Path:
    """In-tree when the tree is writable, else a per-user folder under the temp dir."""
    global _build_dir_cache
    with _lock:
        if _build_dir_cache is None:
            _build_dir_cache = _find_build_dir()
        return _build_dir_cache


def _find_build_dir() -> Path:
    cand = Path(os.environ["FASTLLM_B200_BUILD_DIR"]) if "FASTLLM_B200_BUILD_DIR" in os.environ \
        else Path(__file__).resolve().parent / "_build"
    try:
        cand.mkdir(parents=True, exist_ok=True)
        probe = cand / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return cand
    except OSError:
        alt = Path(tempfile.gettempdir()) / f"fastllm_b200_build_{os.getuid()}"
        alt.mkdir(parents=True, exist_ok=True)
        return alt


def _headers() -> list:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _key(source: Path, defines: dict) -> str:
    h = hashlib.sha256()
    h.update(source.read_bytes())
    for hdr in _headers():
        h.update(hdr.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(ARCH_FLAGS + COMMON_FLAGS).encode())
    return h.hexdigest()[:16]


def library_path(name: str, defines: dict | None = None) -> Path:
    defines = defines or {}
    source = CSRC / f"{name}.cu"
    if not source.exists():
        raise NativeBuildError(f"no CUDA source {source}")
    tag = "".join(f"_{k}{v}" for k, v in sorted(defines.items()))
    return _build_dir() / f"{name}{tag}-{_key(source, defines)}.so"


def _say(msg: str) -> None:
    print(f"[fastllm_b200] {msg}", file=sys.stderr, flush=True)


def compile_library(name: str, defines: dict | None = None, verbose_ptxas: bool = False) -> Path:
    """Build csrc/<name>.cu with the given defines unless it is already built."""
    defines = defines or {}
    out = library_path(name, defines)
    if out.exists():
        return out
    source = CSRC / f"{name}.cu"
    tmp = out.with_suffix(f".tmp{os.getpid()}_{threading.get_ident()}.so")    # one per builder, thread or process
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, f"-I{CSRC}"]
    cmd += [f"-D{k}={v}" for k, v in sorted(defines.items())]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(tmp), str(source)]
    label = name + ("" if not defines else " " + " ".join(f"{k}={v}" for k, v in sorted(defines.items())))
    _say(f"compiling {label} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    # A line now and then while nvcc works, so that a first call does not look hung.
    stop = threading.Event()

    def heartbeat():
        while not stop.wait(10.0):
            _say(f"  still compiling {label} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=heartbeat, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        stop.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise NativeBuildError(f"nvcc failed for {source.name} ({' '.join(cmd)}):\n{log}")
    os.replace(tmp, out)           # atomic: a concurrent builder sees a whole file or none
    tag = "".join(f"_{k}{v}" for k, v in sorted(defines.items()))
    for old in out.parent.glob(f"{name}{tag}-*.so"):        # builds of earlier versions of this source
        if old != out and len(old.name) == len(out.name):
            try:
                old.unlink()
            except OSError:
                pass
    if verbose_ptxas:
        _say(log)
    _say(f"built {out.name} in {time.time() - t0:.1f} s")
    return out


def load_library(name: str, defines: dict | None = None) -> ctypes.CDLL:
    """The ctypes handle of a library, compiling it first if need be."""
    defines = defines or {}
    key = (name, tuple(sorted(defines.items())))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, defines)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise NativeBuildError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
        return lib


def compile_many(jobs: list, workers: int | None = None) -> list:
    """Build several (name, defines) libraries side by side."""
    from concurrent.futures import ThreadPoolExecutor

    unique = {}
    for name, defines in jobs:                      # a library asked for twice is built once
        unique.setdefault((name, tuple(sorted((defines or {}).items()))), (name, defines))
    jobs = list(unique.values())
    workers = workers or min(len(jobs), os.cpu_count() or 4) or 1
    with ThreadPoolExecutor(max_workers=workers) as pool:
        return list(pool.map(lambda j: compile_library(j[0], j[1]), jobs))
