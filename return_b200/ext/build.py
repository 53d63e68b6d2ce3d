"""Compiles the CUDA sources of ``return_b200/csrc`` for sm_100a and loads them with ctypes.

There is no prebuilt binary in a checkout: a library is compiled by ``nvcc`` the first time it
is asked for and kept next to the sources (``csrc/_build``), or, where that folder cannot be
written, under ``$RETURN_B200_BUILD_DIR`` or the system's temporary folder.  The file name
holds a hash of the sources, the flags and the compiler version, so an edit or another
specialisation (``defines``) makes another file.  A kernel library may be specialised for a model
through ``defines`` (the attention kernels take the head size this way), so the first call
compiles what this model needs and nothing else.

While nvcc runs, a line is printed to stderr every few seconds, because the first call of a
program that uses the engine waits for it.
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
from typing import Dict, Iterable, Optional, Sequence

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class ExtensionError(RuntimeError):
    """The CUDA extension could not be compiled or loaded.  The engine has no other path."""


def find_nvcc() -> str:
    for cand in (os.environ.get("RETURN_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise ExtensionError("nvcc was not found (looked at $RETURN_B200_NVCC, $CUDA_HOME/bin, "
                         "/usr/local/cuda/bin and PATH); the engine's kernels cannot be compiled")


_nvcc_version: Optional[str] = None


def nvcc_version() -> str:
    global _nvcc_version
    if _nvcc_version is None:
        out = subprocess.run([find_nvcc(), "--version"], capture_output=True, text=True).stdout
        _nvcc_version = out.strip().splitlines()[-1] if out.strip() else "unknown"
    return _nvcc_version


def build_dir() -> str:
    """A writable folder for the compiled libraries."""
    cands = []
    if os.environ.get("RETURN_B200_BUILD_DIR"):
        cands.append(os.environ["RETURN_B200_BUILD_DIR"])
    cands.append(os.path.join(CSRC, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"return_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise ExtensionError(f"no writable build folder among {cands}")


def _readable_prebuilt(name: str) -> Optional[str]:
    """A library built earlier next to the sources, usable even if that folder is read-only now."""
    path = os.path.join(CSRC, "_build", name)
    return path if os.path.isfile(path) else None


def _source_hash(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for f in list(sources) + headers:
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(flags).encode())
    h.update(nvcc_version().encode())
    return h.hexdigest()[:16]


def _run_with_heartbeat(cmd, what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    stop = threading.Event()

    def beat():
        while not stop.wait(8.0):
            print(f"[return_b200] still compiling {what} ... {time.time() - t0:.0f} s",
                  file=sys.stderr, flush=True)

    th = threading.Thread(target=beat, daemon=True)
    th.start()
    try:
        out, _ = proc.communicate()
    finally:
        stop.set()
    if proc.returncode != 0:
        raise ExtensionError(f"nvcc failed for {what}:\n{' '.join(cmd)}\n{out}")


def library_path(name: str, sources: Sequence[str], defines: Optional[Dict[str, object]] = None,
                 extra_flags: Iterable[str] = ()) -> str:
    """Path of the compiled library, compiling it first if it does not exist yet."""
    defs = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    flags = ARCH_FLAGS + BASE_FLAGS + list(extra_flags) + defs
    tag = _source_hash(sources, flags)
    fname = f"lib{name}-{tag}.so"
    pre = _readable_prebuilt(fname)
    if pre:
        return pre
    out_dir = build_dir()
    out = os.path.join(out_dir, fname)
    if os.path.isfile(out):
        return out
    lock_path = os.path.join(out_dir, f".{fname}.lock")
    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)       # other processes wait here for one compile
        try:
            if os.path.isfile(out):
                return out
            what = name + (" (" + ", ".join(d[2:] for d in defs) + ")" if defs else "")
            print(f"[return_b200] compiling {what} for sm_100a (first use; a minute or so)",
                  file=sys.stderr, flush=True)
            t0 = time.time()
            tmp = out + f".tmp{os.getpid()}"
            cmd = [find_nvcc()] + flags + ["-shared", "-o", tmp] + [os.path.join(CSRC, s) for s in sources]
            _run_with_heartbeat(cmd, what)
            os.replace(tmp, out)
            for old in os.listdir(out_dir):          # builds of earlier sources under the same name, and their lock files, are of no use now
                stale_lib = old.startswith(f"lib{name}-") and old.endswith(".so") and old != fname
                stale_lock = old.startswith(f".lib{name}-") and old.endswith(".so.lock") and old != f".{fname}.lock"
                if stale_lib or stale_lock:
                    try:
                        os.remove(os.path.join(out_dir, old))
                    except OSError:
                        pass
            print(f"[return_b200] compiled {what} in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
    return out


def load(name: str, sources: Sequence[str], defines: Optional[Dict[str, object]] = None,
         extra_flags: Iterable[str] = ()) -> ctypes.CDLL:
    """The compiled library as a ``ctypes.CDLL`` (cached per process)."""
    key = name + repr(sorted((defines or {}).items()))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = library_path(name, sources, defines, extra_flags)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionError(f"cannot load {path}: {e}") from e
            _loaded[key] = lib
        return lib
