"""Builds the CUDA sources under ``csrc/`` into shared libraries, on demand.

Each ``csrc/<name>.cu`` becomes ``<build dir>/<name>-<hash>.so`` with plain
``extern "C"`` launchers; the hash covers the source, the shared headers and
the compiler flags, so an edited file is rebuilt and a stale library is never
loaded.  A name of the form ``file:MACRO=value`` is that source built with the
macro defined (a variant for one head size, say), a library of its own.  Nothing is compiled until a library is first asked for, and a model
asks only for the libraries its parts name (``ensure_built``), so a first
call compiles what that model needs and nothing else.  While compiling, a
line per library goes to stderr.

The build directory is ``csrc/_build`` inside the package when that is
writable, else a per-user folder under the system's temporary directory.
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
from typing import Dict, Iterable, List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--shared",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]

_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.RLock()


class KernelBuildError(RuntimeError):
    pass


def all_sources() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("MLXB_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc not found (set CUDA_HOME or MLXB_NVCC): the CUDA kernels cannot be built")


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _split(name: str):
    """``"file"`` or ``"file:MACRO=value,MACRO=value"``: a source and the macros of one of its variants."""
    src, _, defs = name.partition(":")
    return src, [d for d in defs.split(",") if d]


def _digest(name: str) -> str:
    src, defines = _split(name)
    if not os.path.exists(os.path.join(CSRC, src + ".cu")):
        raise KernelBuildError(f"no kernel source {os.path.join(CSRC, src + '.cu')}")
    h = hashlib.sha1()
    for path in [os.path.join(CSRC, src + ".cu")] + _headers():
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + defines).encode())
    return h.hexdigest()[:12]


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    if _build_dir is not None:
        return _build_dir
    with _lock:
        if _build_dir is None:
            d = os.environ.get("MLXB_BUILD_DIR") or os.path.join(CSRC, "_build")
            try:
                os.makedirs(d, exist_ok=True)
                fd, probe = tempfile.mkstemp(dir=d)
                os.close(fd)
                os.unlink(probe)
            except OSError:
                d = os.path.join(tempfile.gettempdir(), f"mlx_lm_b200-build-{os.getuid()}")
                os.makedirs(d, exist_ok=True)
            _build_dir = d
    return _build_dir


def lib_path(name: str) -> str:
    src, defines = _split(name)
    stem = src + "".join("." + d.replace("=", "_") for d in defines)
    return os.path.join(build_dir(), f"{stem}-{_digest(name)}.so")


def _compile(name: str) -> str:
    out = lib_path(name)
    if os.path.exists(out):
        return out
    stem, defines = _split(name)
    src = os.path.join(CSRC, stem + ".cu")
    if not os.path.exists(src):
        raise KernelBuildError(f"no kernel source {src}")
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [_nvcc()] + NVCC_FLAGS + ["-D" + d for d in defines] + ["-I", CSRC, "-o", tmp, src, "-lcuda"]
    t0 = time.time()
    label = stem + ".cu" + (" with " + ", ".join(defines) if defines else "")
    print(f"[mlx_lm_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {label}:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, out)
    d = os.path.dirname(out)
    prefix = os.path.basename(out).rsplit("-", 1)[0] + "-"
    for f in os.listdir(d):  # drop libraries of older versions of this source
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(d, f) != out:
            try:
                os.unlink(os.path.join(d, f))
            except OSError:
                pass
    print(f"[mlx_lm_b200] compiled {label} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def ensure_built(names: Iterable[str]) -> None:
    """Compile the named sources that are not built yet, in parallel."""
    todo = [n for n in dict.fromkeys(names) if not os.path.exists(lib_path(n))]
    if not todo:
        return
    if len(todo) == 1:
        _compile(todo[0])
        return
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 2)) as ex:
        list(ex.map(_compile, todo))


def load(name: str) -> ctypes.CDLL:
    """The library of ``csrc/<name>.cu``, compiled first if need be."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _libs.get(name)
        if lib is None:
            lib = ctypes.CDLL(_compile(name))
            lib.mlxb_last_error.restype = ctypes.c_char_p
            _libs[name] = lib
    return lib
