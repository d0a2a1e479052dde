"""Compile the CUDA sources of this folder into one shared library for sm_100a.

The library is built with nvcc alone (no Python headers): every entry point is ``extern "C"`` and is
called through ctypes.  It is built on first use, in ``_build/`` beside the sources when that folder
can be written and in a per-user temporary folder otherwise, and rebuilt when a source or a flag
changes.  While nvcc runs, a line is printed every few seconds so that a first call does not look hung.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libcuinfer_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
              "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[cuinfer_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    found = shutil.which("nvcc")
    if found:
        candidates.append(found)
    for c in candidates:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels of cuinfer_b200 cannot be built")


def sources() -> list[str]:
    return sorted(os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("CUINFER_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    local = os.path.join(_HERE, "_build")
    if _writable_dir(local):
        return local
    fallback = os.path.join(tempfile.gettempdir(), f"cuinfer_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"no writable build folder: tried {local} and {fallback}")


def library_path() -> str:
    return os.path.join(build_dir(), LIB_NAME)


def is_current() -> bool:
    d = build_dir()
    stamp = os.path.join(d, "fingerprint")
    lib = os.path.join(d, LIB_NAME)
    if not (os.path.isfile(stamp) and os.path.isfile(lib)):
        return False
    with open(stamp) as fh:
        return fh.read().strip() == _fingerprint()


def _compile_one(nvcc: str, src: str, obj: str) -> tuple[str, float]:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", _HERE, "-c", src, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return src, time.time() - t0


def build(verbose: bool = True, force: bool = False) -> str:
    """Build the library if it is missing or stale; return its path."""
    d = build_dir()
    lock_path = os.path.join(d, ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and is_current():
                return os.path.join(d, LIB_NAME)
            nvcc = find_nvcc()
            srcs = sources()
            if verbose:
                _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {d} (first use; takes a minute or two)")
            t0 = time.time()
            stop = threading.Event()

            def ticker() -> None:
                while not stop.wait(10.0):
                    _log(f"still compiling ... {time.time() - t0:.0f} s")

            if verbose:
                threading.Thread(target=ticker, daemon=True).start()
            try:
                objs = [os.path.join(d, os.path.basename(s)[:-3] + ".o") for s in srcs]
                workers = max(1, min(len(srcs), os.cpu_count() or 1))
                with concurrent.futures.ThreadPoolExecutor(workers) as pool:
                    futs = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
                    for fut in concurrent.futures.as_completed(futs):
                        src, dt = fut.result()
                        if verbose:
                            _log(f"  compiled {os.path.basename(src)} in {dt:.1f} s")
                lib_tmp = os.path.join(d, LIB_NAME + f".tmp{os.getpid()}")
                cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", lib_tmp, *objs]
                proc = subprocess.run(cmd, capture_output=True, text=True)
                if proc.returncode != 0:
                    raise BuildError(f"link failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
                os.replace(lib_tmp, os.path.join(d, LIB_NAME))
                with open(os.path.join(d, "fingerprint"), "w") as fh:
                    fh.write(_fingerprint())
            finally:
                stop.set()
            if verbose:
                _log(f"built {LIB_NAME} in {time.time() - t0:.1f} s")
            return os.path.join(d, LIB_NAME)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
