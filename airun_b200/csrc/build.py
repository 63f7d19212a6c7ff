"""Compiles the CUDA sources for sm_100a with nvcc (and the host-only ``.cpp`` sources with the
C++ compiler) and loads them with ctypes.

Each ``.cu`` or ``.cpp`` file becomes one shared library, built the first time something
needs it and kept next to the sources (``csrc/_build/``; a temporary folder when
the package folder is read-only).  The library name carries a hash of the
source, the shared headers, the flags and the ``-D`` defines, so an edited file
or another specialisation (a head size, say) is rebuilt and a stale library is
never loaded.  While nvcc runs, a line is printed to stderr every few seconds.
There is no fallback: without nvcc or with a failed compile an error is raised.
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
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

_LOCK = threading.Lock()
_LOADED: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("AIRUN_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found: the kernels of airun_b200 are compiled for sm_100a at first use "
                     "(set CUDA_HOME or AIRUN_NVCC)")


HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread", "-ffp-contract=off"]


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return shutil.which(cand) or cand
    raise BuildError("no C++ compiler found (g++, c++ or $CXX): the host core of airun_b200 is compiled at first use")


_BUILD_DIR: Optional[str] = None


def _build_dir() -> str:
    global _BUILD_DIR
    with _LOCK:
        if _BUILD_DIR is not None:
            return _BUILD_DIR
        d = os.environ.get("AIRUN_BUILD_DIR") or os.path.join(CSRC_DIR, "_build")
        try:
            os.makedirs(d, exist_ok=True)
            fd, probe = tempfile.mkstemp(dir=d)
            os.close(fd)
            os.unlink(probe)
        except OSError:
            d = os.path.join(tempfile.gettempdir(), f"airun_b200_build_{os.getuid()}")
            os.makedirs(d, exist_ok=True)
        _BUILD_DIR = d
        return d


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _key(source: str, defines: Sequence[Tuple[str, object]], extra: Sequence[str]) -> str:
    h = hashlib.sha256()
    for p in [source] + _headers():
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode())
            h.update(f.read())
    flags = HOST_FLAGS if source.endswith(".cpp") else (ARCH_FLAGS, BASE_FLAGS)
    h.update(repr((flags, sorted(defines), list(extra))).encode())
    return h.hexdigest()[:16]


def library_path(name: str, defines: Optional[Dict[str, object]] = None,
                 extra_flags: Sequence[str] = ()) -> Tuple[str, str, List[Tuple[str, object]]]:
    source = os.path.join(CSRC_DIR, name + ".cu")
    if not os.path.isfile(source):
        source = os.path.join(CSRC_DIR, name + ".cpp")
    if not os.path.isfile(source):
        raise BuildError(f"source {os.path.join(CSRC_DIR, name)}.cu / .cpp is missing")
    defs = sorted((defines or {}).items())
    tag = "".join(f"_{k}{v}" for k, v in defs)
    return (os.path.join(_build_dir(), f"lib{name}{tag}_{_key(source, defs, extra_flags)}.so"), source, defs)


def compile_command(name: str, defines: Optional[Dict[str, object]] = None,
                    extra_flags: Sequence[str] = (), out: Optional[str] = None) -> List[str]:
    path, source, defs = library_path(name, defines, extra_flags)
    if source.endswith(".cpp"):
        return ([find_cxx()] + HOST_FLAGS + list(extra_flags) + [f"-D{k}={v}" for k, v in defs]
                + ["-I", CSRC_DIR, "-o", out or path, source])
    return ([find_nvcc()] + ARCH_FLAGS + BASE_FLAGS + list(extra_flags)
            + [f"-D{k}={v}" for k, v in defs] + ["-I", CSRC_DIR, "-o", out or path, source])


def build(name: str, defines: Optional[Dict[str, object]] = None,
          extra_flags: Sequence[str] = (), quiet: bool = False) -> str:
    """Makes sure the library of ``name`` exists and returns its path."""
    path, source, defs = library_path(name, defines, extra_flags)
    if os.path.isfile(path):
        return path
    tmp = f"{path}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = compile_command(name, defines, extra_flags, out=tmp)
    label = os.path.basename(source) + ("" if not defs else " " + " ".join(f"{k}={v}" for k, v in defs))
    if not quiet:
        print(f"[airun_b200] compiling {label}" + ("" if source.endswith(".cpp") else " for sm_100a") + " ...",
              file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(8.0):
            print(f"[airun_b200] still compiling {label} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    hb = threading.Thread(target=heartbeat, daemon=True)
    if not quiet:
        hb.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise BuildError(f"{os.path.basename(cmd[0])} failed on {source} (exit {proc.returncode}):\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, path)
    # libraries of older versions of this source with the same defines (the same name, another
    # hash) are of no use any more
    stem = os.path.basename(path).rsplit("_", 1)[0]
    stale = re.compile(re.escape(stem) + r"_[0-9a-f]{16}\.so$")
    for f in os.listdir(os.path.dirname(path)):
        if stale.match(f) and f != os.path.basename(path):
            try:
                os.unlink(os.path.join(os.path.dirname(path), f))
            except OSError:
                pass
    if not quiet:
        print(f"[airun_b200] compiled {label} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return path


def build_many(items: Iterable[Tuple[str, Optional[Dict[str, object]]]], quiet: bool = False) -> List[str]:
    """Builds several libraries side by side (nvcc is single-threaded per file)."""
    items = list(items)
    results: List[Optional[str]] = [None] * len(items)
    errors: List[BaseException] = []

    def work(i: int, name: str, defines):
        try:
            results[i] = build(name, defines, quiet=quiet)
        except BaseException as e:     # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i, n, d)) for i, (n, d) in enumerate(items)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return [r for r in results if r]


def load(name: str, defines: Optional[Dict[str, object]] = None,
         extra_flags: Sequence[str] = ()) -> ctypes.CDLL:
    """The loaded library of ``name`` (compiled first if need be)."""
    path, _, _ = library_path(name, defines, extra_flags)
    with _LOCK:
        if path in _LOADED:
            return _LOADED[path]
    built = build(name, defines, extra_flags)
    with _LOCK:
        if built not in _LOADED:
            _LOADED[built] = ctypes.CDLL(built)
        return _LOADED[built]
