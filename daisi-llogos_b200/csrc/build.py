"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each ``.cu`` file becomes one shared library under ``csrc/_build/`` whose name carries a
hash of its sources, so a changed source is rebuilt and a stale library is never loaded.
A library is compiled when something first needs it (and all of them by ``build_all``);
while nvcc runs, a line is printed every few seconds.  There is no fallback: if a library
cannot be built or loaded, the caller gets the error.

The reference compiles its kernels at run time too, with NVRTC and a disk cache of the PTX
(Daisi.Llogos.Cuda/CudaModule.cs:35-127).
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
from typing import Dict, List

_HERE = os.path.dirname(os.path.abspath(__file__))

# library name -> sources (first is the .cu that is compiled; the rest are hashed with it)
SOURCES: Dict[str, List[str]] = {
    "elementwise": ["elementwise.cu", "common.cuh", "kernel_args.h"],
    "gemm_simt": ["gemm_simt.cu", "common.cuh"],
    "gemm_tc": ["gemm_tc.cu", "common.cuh", "kernel_args.h"],
    "attention_simt": ["attention_simt.cu", "common.cuh", "kernel_args.h", "attention_noalloc.h"],
    "attention_mma": ["attention_mma.cu", "common.cuh", "kernel_args.h"],
    "attention_tc": ["attention_tc.cu", "common.cuh", "kernel_args.h"],
    "attention_decode_tma": ["attention_decode_tma.cu", "common.cuh", "kernel_args.h"],
    "sampling": ["sampling.cu", "common.cuh"],
    "init": ["init.cu", "common.cuh"],
    "block_runner": ["block_runner.cu", "kernel_args.h"],
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--extended-lambda", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# Further flags for a build of its own, e.g. LLOGOS_NVCC_FLAGS=-DLLG_STAMPS for the kernels' time stamps (common.cuh):
# they are part of the library's name, so such a build lies beside the ordinary one and neither replaces the other.
_EXTRA_FLAGS = [f for f in os.environ.get("LLOGOS_NVCC_FLAGS", "").split() if f]
NVCC_FLAGS += _EXTRA_FLAGS
_VARIANT = ("." + hashlib.sha256(" ".join(_EXTRA_FLAGS).encode()).hexdigest()[:6]) if _EXTRA_FLAGS else ""

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("LLOGOS_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $LLOGOS_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no other path")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for src in SOURCES[name]:
        with open(os.path.join(_HERE, src), "rb") as f:
            h.update(src.encode() + b"\0" + f.read() + b"\0")
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"llogos_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"libllogos_{name}{_VARIANT}-{_digest(name)}.so")


def _say(msg: str) -> None:
    print(f"[llogos build] {msg}", file=sys.stderr, flush=True)


def compile_library(name: str, *, verbose: bool = True) -> str:
    """Build ``name`` if its library is missing; returns the library's path."""
    if name not in SOURCES:
        raise BuildError(f"no CUDA library named '{name}' (known: {', '.join(sorted(SOURCES))})")
    out = library_path(name)
    if os.path.isfile(out):
        return out
    lock_path = out + ".lock"
    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if os.path.isfile(out):
                return out
            tmp = f"{out}.{os.getpid()}.tmp"
            cmd = [_nvcc(), *NVCC_FLAGS, "-o", tmp, os.path.join(_HERE, SOURCES[name][0])]
            if verbose:
                _say(f"compiling {SOURCES[name][0]} for sm_100a ...")
            t0 = time.time()
            env = dict(os.environ)
            env.setdefault("TMPDIR", tempfile.gettempdir())
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=_HERE, env=env)
            beat = 0
            while True:
                try:
                    proc.wait(timeout=5)
                    break
                except subprocess.TimeoutExpired:
                    beat += 1
                    if verbose:
                        _say(f"  still compiling {SOURCES[name][0]} ({int(time.time() - t0)} s)")
            log = proc.stdout.read().decode("utf-8", "replace")
            if proc.returncode != 0 or not os.path.isfile(tmp):
                if os.path.exists(tmp):
                    os.unlink(tmp)
                raise BuildError(f"nvcc failed on {SOURCES[name][0]} (exit {proc.returncode}):\n{log}")
            os.replace(tmp, out)
            if verbose:
                _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
            # libraries of older source versions are of no use any more
            prefix = f"libllogos_{name}{_VARIANT}-"
            for f in os.listdir(os.path.dirname(out)):
                if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(out):
                    try:
                        os.unlink(os.path.join(os.path.dirname(out), f))
                    except OSError:
                        pass
            return out
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
            try:
                os.unlink(lock_path)
            except OSError:
                pass


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library ``name``, compiled first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
            lib.llg_last_error.restype = ctypes.c_char_p
            lib.llg_last_error.argtypes = []
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    return [compile_library(n, verbose=verbose) for n in SOURCES]
