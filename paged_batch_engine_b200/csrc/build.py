"""Compiles the CUDA sources of this package for sm_100a and loads them with ctypes.

Every kernel file exports plain C entry points (pointers, sizes and a stream), so a
library is built by one ``nvcc`` call without any framework header, in seconds, and is
loaded without an import hook.  Libraries are built in-tree under ``csrc/_build`` (kept
out of version control) the first time they are asked for; a file whose source, headers,
flags or compile-time constants (the head size of an attention kernel, for instance)
change gets a new name, so a stale binary is never loaded.  Only what a model needs is
compiled: the attention kernels for its head sizes, not for every size.

There is no fallback: if ``nvcc`` is missing or a compile fails, the error is raised.
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
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

KERNEL_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("PBE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (looked at $PBE_NVCC, PATH and /usr/local/cuda/bin): the CUDA "
                     "kernels of this engine cannot be built and there is no other code path")


_build_dir: Optional[str] = None


def build_dir() -> str:
    """In-tree ``csrc/_build``; a per-user temporary folder when the tree is read-only."""
    global _build_dir
    with _lock:
        if _build_dir is None:
            _build_dir = _find_build_dir()
        return _build_dir


def _find_build_dir() -> str:
    d = os.environ.get("PBE_BUILD_DIR") or os.path.join(os.path.dirname(KERNEL_DIR), "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"pbe_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers() -> List[str]:
    return sorted(os.path.join(KERNEL_DIR, n) for n in os.listdir(KERNEL_DIR) if n.endswith((".cuh", ".h")))


def _included_sources(source: str, seen: Optional[set] = None) -> List[str]:
    """Files of the kernel folder that ``source`` pulls in with ``#include "..."`` and that are
    not headers (one library compiles another's .cu into itself), recursively."""
    seen = set() if seen is None else seen
    out: List[str] = []
    with open(source, "r", errors="replace") as f:
        for line in f:
            line = line.strip()
            if line.startswith("#include") and '"' in line:
                name = line.split('"')[1]
                path = os.path.join(KERNEL_DIR, name)
                if not name.endswith((".cuh", ".h")) and os.path.isfile(path) and path not in seen:
                    seen.add(path)
                    out.append(path)
                    out += _included_sources(path, seen)
    return out


def _key(source: str, defines: Dict[str, object], extra: Sequence[str]) -> str:
    h = hashlib.sha256()
    for path in [source] + _included_sources(source) + _headers():
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(ARCH_FLAGS + NVCC_FLAGS + list(extra)).encode())
    return h.hexdigest()[:16]


def library_path(name: str, defines: Optional[Dict[str, object]] = None,
                 extra_flags: Sequence[str] = ()) -> Tuple[str, str]:
    defines = dict(defines or {})
    source = os.path.join(KERNEL_DIR, name + ".cu")
    if not os.path.isfile(source):
        raise BuildError(f"no kernel source {source}")
    tag = "".join(f"_{k.lower().replace('pbe_', '')}{v}" for k, v in sorted(defines.items()))
    fname = f"libpbe_{name}{tag}-{_key(source, defines, extra_flags)}.so"
    return source, os.path.join(build_dir(), fname)


def _drop_older_builds(out: str) -> None:
    """After a build: libraries of the same name and defines made from earlier sources (same file
    name up to the hash) are of no use any more and only grow the build folder."""
    folder, fname = os.path.split(out)
    stem = fname[:fname.rfind("-") + 1]
    try:
        for other in os.listdir(folder):
            if other != fname and other.startswith(stem) and other.endswith(".so") and \
                    len(other) == len(fname):
                try:
                    os.remove(os.path.join(folder, other))
                except OSError:
                    pass
    except OSError:
        pass


def compile_library(name: str, defines: Optional[Dict[str, object]] = None,
                    extra_flags: Sequence[str] = (), verbose: bool = True) -> str:
    """Build one library if it is not there yet; returns its path."""
    source, out = library_path(name, defines, extra_flags)
    if os.path.isfile(out):
        return out
    cmd = [_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + list(extra_flags) + ["-I", KERNEL_DIR]
    cmd += [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tmp = f"{out}.tmp{os.getpid()}.{threading.get_ident()}"
    cmd += ["-o", tmp, source]
    label = os.path.basename(out)
    if verbose:
        print(f"[pbe] compiling {label} ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            if verbose:
                print(f"[pbe] still compiling {label} ({time.time() - t0:.0f} s)", file=sys.stderr,
                      flush=True)
    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed for {source} ({' '.join(cmd)}):\n{log}")
    os.replace(tmp, out)
    _drop_older_builds(out)
    if verbose:
        print(f"[pbe] built {label} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


_by_request: Dict[tuple, ctypes.CDLL] = {}


def load_library(name: str, defines: Optional[Dict[str, object]] = None,
                 extra_flags: Sequence[str] = ()) -> ctypes.CDLL:
    # the sources are hashed once per (name, defines) and process, not once per call
    request = (name, tuple(sorted((defines or {}).items())), tuple(extra_flags))
    lib = _by_request.get(request)
    if lib is not None:
        return lib
    lib = _load_library(name, defines, extra_flags)
    _by_request[request] = lib
    return lib


def _load_library(name: str, defines: Optional[Dict[str, object]] = None,
                  extra_flags: Sequence[str] = ()) -> ctypes.CDLL:
    _, out = library_path(name, defines, extra_flags)
    with _lock:
        lib = _loaded.get(out)
        if lib is not None:
            return lib
    path = compile_library(name, defines, extra_flags)
    with _lock:
        lib = _loaded.get(path)
        if lib is None:
            lib = ctypes.CDLL(path)
            _loaded[path] = lib
        return lib


def compile_many(jobs: Iterable[Tuple[str, Optional[Dict[str, object]]]], workers: int = 0) -> List[str]:
    """Build several libraries side by side (used by the build check and before a model's
    first step so that its kernels compile in parallel)."""
    jobs = list(jobs)
    workers = workers or min(len(jobs), os.cpu_count() or 4) or 1
    with ThreadPoolExecutor(max_workers=workers) as ex:
        return list(ex.map(lambda j: compile_library(j[0], j[1]), jobs))


# ------------------------------------------------------------------ host libraries (plain C++)
HOST_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "host")
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def load_host_library(name: str) -> ctypes.CDLL:
    """Builds (g++, once) and loads a host-side C++ library of the package: the runtime parts
    that need no GPU.  Same naming and caching rule as the CUDA libraries."""
    source = os.path.join(HOST_DIR, name + ".cpp")
    if not os.path.isfile(source):
        raise BuildError(f"no host source {source}")
    h = hashlib.sha256()
    for path in [source] + _headers():            # host sources may include the kernels' plain structs
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(repr(HOST_FLAGS).encode())
    out = os.path.join(build_dir(), f"libpbe_host_{name}-{h.hexdigest()[:16]}.so")
    with _lock:
        lib = _loaded.get(out)
        if lib is not None:
            return lib
    if not os.path.isfile(out):
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found (g++): the host runtime of this engine cannot be built")
        tmp = f"{out}.tmp{os.getpid()}.{threading.get_ident()}"
        print(f"[pbe] compiling {os.path.basename(out)} ...", file=sys.stderr, flush=True)
        proc = subprocess.run([cxx] + HOST_FLAGS + ["-o", tmp, source], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise BuildError(f"{cxx} failed for {source}:\n{proc.stdout}")
        os.replace(tmp, out)
        _drop_older_builds(out)
    with _lock:
        lib = _loaded.get(out)
        if lib is None:
            lib = ctypes.CDLL(out)
            _loaded[out] = lib
        return lib
