"""Compiles the package's CUDA sources for sm_100a with nvcc and caches the result.

Each source file under ``redline_b200/csrc`` becomes one shared object of plain
extern "C" launchers (no torch headers, so a file compiles in seconds).  An object
is keyed by the hash of its sources and flags: ``<name>-<key>.so``.  Objects live in
``redline_b200/csrc/_build`` when that folder can be written, else in a per-user
folder under the system's temporary directory, so that a read-only checkout run by
another user still works.  Head size and the like are passed as ``-D`` flags: a
model compiles only the variants it needs, at its first call, and a line is
printed now and then meanwhile.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Optional, Tuple

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]

_lock = threading.Lock()
_build_dir: Optional[str] = None


class BuildError(RuntimeError):
    pass


def nvcc_path() -> str:
    for cand in (os.environ.get("REDLINE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of redline_b200 cannot be built "
                     "(set REDLINE_NVCC or put nvcc on PATH)")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    global _build_dir
    if _build_dir is None:
        cands = []
        if os.environ.get("REDLINE_BUILD_DIR"):
            cands.append(os.environ["REDLINE_BUILD_DIR"])
        cands.append(os.path.join(CSRC, "_build"))
        cands.append(os.path.join(tempfile.gettempdir(), f"redline_b200_build_{os.getuid()}"))
        for c in cands:
            if _writable_dir(c):
                _build_dir = c
                break
        else:
            raise BuildError("no writable folder for compiled kernels; tried " + ", ".join(cands))
    return _build_dir


def _hash(sources: Iterable[str], flags: Iterable[str]) -> str:
    h = hashlib.sha256()
    for s in sources:
        with open(s, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def module_path(name: str, source: str, defines: Optional[Dict[str, object]] = None,
                extra_flags: Optional[List[str]] = None) -> Tuple[str, List[str], str]:
    src = os.path.join(CSRC, source)
    flags = list(ARCH_FLAGS) + list(BASE_FLAGS) + [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    flags += list(extra_flags or [])
    key = _hash([src] + _headers(), flags)
    return os.path.join(build_dir(), f"{name}-{key}.so"), flags, src


def compile_module(name: str, source: str, defines: Optional[Dict[str, object]] = None,
                   extra_flags: Optional[List[str]] = None, verbose: bool = True) -> str:
    """Returns the path of the shared object for (source, defines), compiling it if needed."""
    out, flags, src = module_path(name, source, defines, extra_flags)
    if os.path.exists(out):
        return out
    with _lock:
        if os.path.exists(out):
            return out
        tmp = f"{out}.{os.getpid()}.tmp"
        cmd = [nvcc_path()] + flags + ["-I", CSRC, "-o", tmp, src]
        t0 = time.time()
        if verbose:
            print(f"[redline_b200] compiling {name} for sm_100a ...", file=sys.stderr, flush=True)
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        done = threading.Event()

        def ticker():
            while not done.wait(10.0):
                print(f"[redline_b200] still compiling {name} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

        th = threading.Thread(target=ticker, daemon=True)
        if verbose:
            th.start()
        log, _ = proc.communicate()
        done.set()
        if proc.returncode != 0:
            if os.path.exists(tmp):
                os.unlink(tmp)
            raise BuildError(f"nvcc failed for {source} ({' '.join(cmd)}):\n{log}")
        os.replace(tmp, out)
        if verbose:
            print(f"[redline_b200] compiled {name} in {time.time() - t0:.1f} s -> {out}",
                  file=sys.stderr, flush=True)
    return out


def remove_other_versions(paths: Iterable[str]) -> None:
    """Deletes, next to each of the given built files ``<module>-<key>.so``, the files of the same module
    with another key (built from other versions of the sources; nothing loads them any more)."""
    for path in paths:
        folder, name = os.path.split(path)
        module = name.rsplit("-", 1)[0]
        for other in os.listdir(folder):
            if other != name and other.endswith(".so") and other.rsplit("-", 1)[0] == module:
                try:
                    os.remove(os.path.join(folder, other))
                except OSError:
                    pass

