"""Builds libgemmars_b200.so, the C API (include/gemmars_b200.h), with the host compiler.

    python -m gemmars_b200.capi.build        prints the library's path

The library embeds the Python installation that builds it (its executable is compiled in as the
default of GEMMARS_B200_PYTHON) and links against that installation's libpython.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
INCLUDE = os.path.join(ROOT, "include")
LIB_NAME = "libgemmars_b200.so"


class CapiBuildError(RuntimeError):
    pass


def build_dir() -> str:
    """Beside the sources when that folder can be written, else a per-user temporary folder."""
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        if os.access(d, os.W_OK):
            return d
    except OSError:
        pass
    d = os.path.join(tempfile.gettempdir(), f"gemmars_b200_capi_{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def _command(out: str) -> list:
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    version = sysconfig.get_config_var("LDVERSION") or sysconfig.get_config_var("VERSION")
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", "-shared", "-fPIC", "-fvisibility=default",
           f"-I{INCLUDE}", f"-I{sysconfig.get_paths()['include']}",
           f'-DGB_PYTHON_EXECUTABLE="{sys.executable}"', f'-DGB_DEFAULT_HOME="{ROOT}"',
           os.path.join(HERE, "capi.cpp"), "-o", out]
    if libdir:
        cmd += [f"-L{libdir}", f"-Wl,-rpath,{libdir}"]
    return cmd + [f"-lpython{version}", "-ldl", "-lpthread"]


def library() -> str:
    """The path of the built library; compiled first when it is not there or its sources changed."""
    h = hashlib.sha256()
    for path in (os.path.join(HERE, "capi.cpp"), os.path.join(INCLUDE, "gemmars_b200.h")):
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(_command("")).encode())
    folder = os.path.join(build_dir(), h.hexdigest()[:12])
    out = os.path.join(folder, LIB_NAME)
    if not os.path.exists(out):
        os.makedirs(folder, exist_ok=True)
        tmp = f"{out}.{os.getpid()}.tmp"
        print(f"[gemmars_b200] compiling {LIB_NAME} (first use)", file=sys.stderr, flush=True)
        proc = subprocess.run(_command(tmp), capture_output=True, text=True)
        if proc.returncode != 0:
            raise CapiBuildError(f"the C API did not compile:\n{' '.join(_command(tmp))}\n{proc.stdout}{proc.stderr}")
        os.replace(tmp, out)
    return out


if __name__ == "__main__":
    print(library())
