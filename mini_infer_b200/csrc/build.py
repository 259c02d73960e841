"""Compile the CUDA sources for sm_100a and load them as shared objects.

Each ``.cu`` file becomes one shared object with ``extern "C"`` entry points, loaded
with :mod:`ctypes`.  A library is compiled the first time something asks for it (so a
run compiles only the kernels it uses) and is cached under ``csrc/_build`` with a hash
of its sources and flags in the file name; when that folder cannot be written, a
per-user folder under the system's temporary directory is used instead.  While nvcc
runs, a progress line goes to stderr every few seconds.

There is no fallback: if nvcc is missing or a compile fails, the caller gets a
``KernelBuildError`` that says so.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]

# library name -> (sources, extra headers that invalidate the cache, extra flags)
LIBRARIES: dict[str, tuple[list[str], list[str], list[str]]] = {
    "elementwise": (["elementwise.cu"], ["common.cuh"], []),
    "gemm_f32": (["gemm_f32.cu"], ["common.cuh"], []),
    "attention_generic": (["attention_generic.cu"], ["common.cuh"], []),
    "sampling": (["sampling.cu"], ["common.cuh"], []),
    "attention_mma": (["attention_mma.cu"], ["common.cuh", "attention_noalloc.h"], []),
    "gemm_tma": (["gemm_tma.cu"], ["common.cuh"], []),
    "attention_tc": (["attention_tc.cu"], ["common.cuh"], []),
}


class KernelBuildError(RuntimeError):
    pass


_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def register_library(name: str, sources: list[str], headers: list[str] | None = None,
                     flags: list[str] | None = None) -> None:
    """Add a library (paths relative to ``csrc`` or absolute)."""
    LIBRARIES[name] = (list(sources), list(headers or []), list(flags or []))


def find_nvcc() -> str:
    for env in ("MINI_INFER_NVCC",):
        p = os.environ.get(env)
        if p and os.path.isfile(p):
            return p
    for env in ("CUDA_HOME", "CUDA_PATH"):
        root = os.environ.get(env)
        if root and os.path.isfile(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    p = shutil.which("nvcc")
    if p:
        return p
    if os.path.isfile("/usr/local/cuda/bin/nvcc"):
        return "/usr/local/cuda/bin/nvcc"
    raise KernelBuildError(
        "nvcc was not found (looked at MINI_INFER_NVCC, CUDA_HOME, PATH, /usr/local/cuda); "
        "the engine's kernels must be compiled for sm_100a and there is no fallback"
    )


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("MINI_INFER_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    in_tree = os.path.join(CSRC_DIR, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"mini_infer_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise KernelBuildError(f"neither {in_tree} nor {fallback} can be written")


def _abs(path: str) -> str:
    return path if os.path.isabs(path) else os.path.join(CSRC_DIR, path)


def _digest(name: str) -> str:
    sources, headers, flags = LIBRARIES[name]
    h = hashlib.sha256()
    for f in sources + headers:
        with open(_abs(f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libmi_{name}_{_digest(name)}.so")


def _say(msg: str) -> None:
    print(f"[mini_infer_b200] {msg}", file=sys.stderr, flush=True)


def compile_library(name: str, *, force: bool = False, verbose: bool = True) -> str:
    """Compile ``name`` if its shared object is not there yet; return the path."""
    if name not in LIBRARIES:
        raise KernelBuildError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    out = library_path(name)
    if os.path.isfile(out) and not force:
        return out
    nvcc = find_nvcc()
    sources, _headers, flags = LIBRARIES[name]
    lock_path = os.path.join(os.path.dirname(out), f".{name}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(out) and not force:
                return out
            tmp = f"{out}.{os.getpid()}.tmp"
            cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *flags, "-I", CSRC_DIR, "-o", tmp,
                   *[_abs(s) for s in sources]]
            if verbose:
                _say(f"compiling {name} ({', '.join(sources)}) for sm_100a ...")
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            done = threading.Event()

            def ticker() -> None:
                while not done.wait(5.0):
                    if verbose:
                        _say(f"  still compiling {name} ({time.time() - t0:.0f} s)")

            th = threading.Thread(target=ticker, daemon=True)
            th.start()
            output, _ = proc.communicate()
            done.set()
            if proc.returncode != 0:
                try:
                    os.unlink(tmp)
                except OSError:
                    pass
                raise KernelBuildError(f"nvcc failed for {name} (exit {proc.returncode}):\n{output}")
            os.replace(tmp, out)
            # builds of older versions of the sources are of no use any more
            for stale in os.listdir(os.path.dirname(out)):
                if stale.startswith(f"libmi_{name}_") and stale.endswith(".so") and stale != os.path.basename(out):
                    try:
                        os.unlink(os.path.join(os.path.dirname(out), stale))
                    except OSError:
                        pass
            if verbose:
                _say(f"compiled {name} in {time.time() - t0:.1f} s")
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def library(name: str) -> ctypes.CDLL:
    """The loaded library ``name`` (compiled first when needed)."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            lib.mi_error_message.restype = ctypes.c_char_p
            _loaded[name] = lib
    return lib


def build_all(verbose: bool = True) -> dict[str, str]:
    """Compile every registered library (used by the build check)."""
    return {name: compile_library(name, verbose=verbose) for name in sorted(LIBRARIES)}
