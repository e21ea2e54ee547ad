"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Every `.cu` file becomes one shared library with plain C entry points, built
by `nvcc` on first use and loaded through `ctypes`.  Libraries are kept in
`_build/` beside the sources, named by a hash of the source, the shared header
and the flags, so an edited kernel is rebuilt and a stale one is never
loaded.  If that folder cannot be written (a read-only checkout) a per-user
folder under the system's temporary directory is used instead.  Nothing here
needs a home directory or a network.

There is no fallback: if a library can be neither found nor built, the
caller gets an error that says which and why.
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

_HERE = os.path.dirname(os.path.abspath(__file__))
_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
          "-shared", "-Xcompiler", "-fPIC"]
_FLAGS += os.environ.get("KVAD_NVCC_FLAGS", "").split()      # more flags for every library (part of a build's name)
#: every kernel library of the package, in the order `build_all` compiles them
LIBRARIES = ("rows", "linear_simt", "attention_simt", "sampling", "linear_tcgen05", "linear_rows", "linear_rows_f32",
             "attention_prefill", "attention_decode")

_registered: dict[str, str] = {}       # kernel sources from outside the package: name -> path of the .cu file
_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[kvad_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("KVAD_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $KVAD_NVCC, $CUDA_HOME/bin, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of kvad_b200 cannot be built and there is no other path")


_dir_cache: list[str] = []


def _build_dir() -> str:
    with _dir_lock:
        if not _dir_cache:
            _dir_cache.append(_find_build_dir())
        return _dir_cache[0]


def _find_build_dir() -> str:
    override = os.environ.get("KVAD_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(_HERE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"kvad_b200-build-{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".write-{os.getpid()}-{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable folder for compiled kernels (tried {candidates})")


def register_source(name: str, path: str) -> None:
    """A kernel source from outside the package (a part that brings its own kernel): compiled with
    the same flags and with this folder on the include path, kept in the same build folder."""
    if name in LIBRARIES:
        raise BuildError(f"`{name}` is one of the package's own kernel libraries")
    path = os.path.abspath(path)
    if not os.path.isfile(path):
        raise BuildError(f"no kernel source {path}")
    with _lock:
        if _registered.get(name) not in (None, path):
            _loaded.pop(name, None)
        _registered[name] = path


def registered_sources() -> dict[str, str]:
    return dict(_registered)


def _source_path(name: str) -> str:
    return _registered.get(name) or os.path.join(_HERE, name + ".cu")


def sources() -> list[str]:
    return [n for n in LIBRARIES if os.path.isfile(os.path.join(_HERE, n + ".cu"))] + list(_registered)


def _digest(name: str) -> str:
    h = hashlib.sha256()
    headers = sorted(fn for fn in os.listdir(_HERE) if fn.endswith((".cuh", ".h")))
    for fn in (_source_path(name), *(os.path.join(_HERE, x) for x in headers)):
        with open(fn, "rb") as f:
            h.update(f.read())
    h.update(" ".join(_FLAGS).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"libkvad_{name}.{_digest(name)}.so")


def compile_library(name: str, *, verbose: bool = True) -> str:
    """Builds one library if it is not built yet; returns its path."""
    src = _source_path(name)
    if not os.path.isfile(src):
        raise BuildError(f"no kernel source {src}")
    target = library_path(name)
    if os.path.isfile(target):
        return target
    nvcc = _nvcc()
    tmp = f"{target}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc, *_FLAGS, "-I", _HERE, "-o", tmp, src]
    if verbose:
        _say(f"compiling {os.path.basename(src)} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=_HERE)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            if verbose:
                _say(f"... still compiling {name}.cu ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{out}")
    os.replace(tmp, target)
    for old in ([] if os.environ.get("KVAD_NVCC_FLAGS") else os.listdir(os.path.dirname(target))):   # builds of earlier versions of this source
        if old.startswith(f"libkvad_{name}.") and old.endswith(".so") and old != os.path.basename(target):
            try:
                os.remove(os.path.join(os.path.dirname(target), old))
            except OSError:
                pass
    if verbose:
        _say(f"compiled {name}.cu in {time.time() - t0:.1f} s")
    return target


def build_all(names=None, *, verbose: bool = True) -> dict[str, str]:
    """Builds the given libraries (default: all) side by side."""
    names = list(names) if names is not None else sources()
    todo = [n for n in names if not os.path.isfile(library_path(n))]
    if todo and verbose:
        _say(f"building {len(todo)} kernel librar{'y' if len(todo) == 1 else 'ies'}: {', '.join(todo)}")
    with ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 1))) as pool:
        list(pool.map(lambda n: compile_library(n, verbose=verbose), todo))
    return {n: library_path(n) for n in names}


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name`, compiling it first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        path = compile_library(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from None
        lib.kvad_last_error.restype = ctypes.c_char_p
        lib.kvad_last_error.argtypes = []
        _loaded[name] = lib
        return lib


def loaded_paths() -> list[str]:
    return [lib._name for lib in _loaded.values()]
