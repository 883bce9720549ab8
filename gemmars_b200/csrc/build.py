"""Compiles the package's CUDA sources for sm_100a and loads them through ``ctypes``.

Each ``.cu`` file of this folder is a *unit* that becomes one shared library with ``extern "C"``
entry points taking raw device pointers and a stream.  A unit is compiled the first time it is
asked for, with ``nvcc`` alone (no PyTorch headers), into ``_build/`` beside the sources (or a
per-user folder under the temporary directory when that is not writable).  The library's file
name carries a hash of the sources and flags, so a changed source is compiled again and a
library that is there is simply loaded.  While ``nvcc`` runs, a line is printed every few
seconds.

There is no fallback: a unit that cannot be compiled or loaded raises ``KernelBuildError``.
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
from typing import Dict, Iterable, Optional, Sequence, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): "
                           "the CUDA kernels of gemmars_b200 cannot be built")


def build_dir() -> str:
    d = os.environ.get("GEMMARS_B200_BUILD_DIR") or os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        open(probe, "w").close()
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"gemmars_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers_digest() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(HERE)):
        if name.endswith((".cuh", ".h")):
            with open(os.path.join(HERE, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    return h.hexdigest()


def library_path(unit: str, defines: Sequence[Tuple[str, object]] = ()) -> Tuple[str, list]:
    src = os.path.join(HERE, unit + ".cu")
    if not os.path.exists(src):
        raise KernelBuildError(f"no CUDA source {src}")
    flags = ARCH_FLAGS + BASE_FLAGS + [f"-D{k}={v}" for k, v in defines]
    h = hashlib.sha256()
    with open(src, "rb") as f:
        h.update(f.read())
    h.update(_headers_digest().encode())
    h.update(" ".join(flags).encode())
    tag = "_".join(f"{k.lower()}{v}" for k, v in defines)
    name = f"{unit}{'_' + tag if tag else ''}_{h.hexdigest()[:12]}.so"
    return os.path.join(build_dir(), name), flags


def _compile(unit: str, out: str, flags: list, verbose_ptxas: bool = False) -> None:
    src = os.path.join(HERE, unit + ".cu")
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc()] + flags + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-I", HERE, "-o", tmp, src]
    print(f"[gemmars_b200] compiling {os.path.basename(out)} for sm_100a (first use)", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def tick():
        while not done.wait(10.0):
            print(f"[gemmars_b200] still compiling {unit} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    th = threading.Thread(target=tick, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed for {unit}.cu:\n{' '.join(cmd)}\n{log}")
    if verbose_ptxas:
        print(log, file=sys.stderr)
    os.replace(tmp, out)
    print(f"[gemmars_b200] compiled {unit} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def load(unit: str, defines: Sequence[Tuple[str, object]] = ()) -> ctypes.CDLL:
    """The loaded library of ``unit`` built with ``defines``; compiled first if it is not there."""
    defines = tuple(defines)
    path, flags = library_path(unit, defines)
    with _lock:
        lib = _loaded.get(path)
        if lib is not None:
            return lib
        if not os.path.exists(path):
            _compile(unit, path, flags)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from None
        _loaded[path] = lib
        return lib


def loaded() -> Dict[str, ctypes.CDLL]:
    """The libraries loaded so far, by path."""
    with _lock:
        return dict(_loaded)


PDL_DEFINE = ("GB_PDL", 1)
_pdl = [False]


def set_pdl(on: bool) -> None:
    """Whether the next launches use the units' builds with programmatic dependent launch (a kernel
    may start under the one before it).  The engine turns it on for prompt steps."""
    _pdl[0] = bool(on)


def pdl() -> bool:
    return _pdl[0]


def ensure(units: Iterable[Tuple[str, Sequence[Tuple[str, object]]]], jobs: Optional[int] = None) -> None:
    """Compiles, in parallel, those of ``units`` ((unit, defines) pairs) that are not built yet."""
    todo = []
    for unit, defines in units:
        for variant in (tuple(defines), tuple(defines) + (PDL_DEFINE,)):   # both builds: see set_pdl
            path, flags = library_path(unit, variant)
            if not os.path.exists(path) and (unit, path) not in [(u, p) for u, p, _ in todo]:
                todo.append((unit, path, flags))
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=jobs or min(len(todo), os.cpu_count() or 4)) as ex:
        for f in [ex.submit(_compile, u, p, fl) for u, p, fl in todo]:
            f.result()
