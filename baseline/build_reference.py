"""Builds the reference arm of the benchmark: the UNMODIFIED engine sources of typr7/cuInfer plus a small driver.

The reference's CMake build fetches nlohmann_json, pybind11, libzmq, cppzmq and msgpack from GitHub, which an
offline machine cannot do.  Only ``csrc/engine/engine_core.cpp`` (the ZeroMQ loop) and the pybind module need
those; every other file of ``CMakeLists.txt:16-57`` compiles with nvcc and g++ alone, given
  * ``nlohmann/json.hpp`` (header-only; a copy ships inside an installed Python package), and
  * a ``msgpack.hpp`` that defines the two macros ``csrc/engine/protocol.h`` uses as no-ops (the structs are then
    plain structs; nothing is serialised without the socket).
This script copies ``csrc/`` unchanged into ``baseline/_ref/csrc``, compiles it for sm_100a into
``baseline/_ref/obj`` and links ``baseline/reference_bench.cpp`` (the engine loop without the socket) into
``baseline/_ref/bin/reference_bench``.  ``baseline/_ref`` is not part of the repository's history.

    python baseline/build_reference.py [--source /path/to/reference] [--jobs N] [--force]
"""
from __future__ import annotations

import argparse
import concurrent.futures
import glob
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
BINARY = os.path.join(REF, "bin", "reference_bench")
DRIVER = os.path.join(HERE, "reference_bench.cpp")
STAMP = os.path.join(REF, "bin", "reference_bench.stamp")

# CMakeLists.txt:16-57 of the reference without csrc/engine/engine_core.cpp
SOURCE_GLOBS = ("common/*.cpp", "cuda/*.cpp", "scheduler/*.cpp", "executor/*.cpp", "model/*.cpp",
                "model/layers/*.cpp", "ops/*.cu")

MSGPACK_STUB = """#pragma once
// Stand-in for msgpack-cxx: the reference's protocol structs only use these two macros.
#define MSGPACK_DEFINE_MAP(...)
#define MSGPACK_ADD_ENUM(...)
"""


def find_json_header() -> str | None:
    for base in sys.path + ["/usr/include", "/usr/local/include"]:
        if not base or not os.path.isdir(base):
            continue
        for pattern in ("nlohmann/json.hpp", "include/nlohmann/json.hpp", "include/*/thirdparty/nlohmann/json.hpp",
                        "*/include/nlohmann/json.hpp", "*/include/*/thirdparty/nlohmann/json.hpp"):
            hits = glob.glob(os.path.join(base, pattern))
            if hits:
                return hits[0]
    return None


def sources(csrc: str) -> list[str]:
    out = []
    for pattern in SOURCE_GLOBS:
        out += sorted(glob.glob(os.path.join(csrc, pattern)))
    return out


def fingerprint(csrc: str) -> str:
    h = hashlib.sha256()
    for path in sources(csrc) + sorted(glob.glob(os.path.join(csrc, "**", "*.h"), recursive=True)) + [DRIVER]:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def is_built() -> bool:
    csrc = os.path.join(REF, "csrc")
    if not (os.path.exists(BINARY) and os.path.exists(STAMP) and os.path.isdir(csrc)):
        return False
    with open(STAMP) as fh:
        return fh.read().strip() == fingerprint(csrc)


def run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd[:6])} ... failed:\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")


def build(source: str | None = None, jobs: int = 0, force: bool = False) -> str:
    """Returns the path of the binary; raises RuntimeError with the compiler's message when something fails."""
    csrc = os.path.join(REF, "csrc")
    if not os.path.isdir(csrc):
        source = source or os.environ.get("CUINFER_REFERENCE_SOURCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
        if not os.path.isdir(os.path.join(source, "csrc")):
            raise RuntimeError(f"the reference's sources are not at {source} and no copy is under baseline/_ref/csrc")
        os.makedirs(REF, exist_ok=True)
        shutil.copytree(os.path.join(source, "csrc"), csrc)
        for folder, _, _ in os.walk(csrc):          # a read-only checkout gives read-only folders
            os.chmod(folder, 0o755)
    if not force and is_built():
        return BINARY
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found")
    stub = os.path.join(REF, "stub")
    os.makedirs(os.path.join(stub, "nlohmann"), exist_ok=True)
    with open(os.path.join(stub, "msgpack.hpp"), "w") as fh:
        fh.write(MSGPACK_STUB)
    json_copy = os.path.join(stub, "nlohmann", "json.hpp")
    if not os.path.exists(json_copy):
        header = find_json_header()
        if header is None:
            raise RuntimeError("nlohmann/json.hpp not found on this machine")
        shutil.copyfile(header, json_copy)
    obj_dir = os.path.join(REF, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    os.makedirs(os.path.dirname(BINARY), exist_ok=True)
    flags = ["-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-w",
             f"-I{csrc}", f"-I{stub}"]
    units = [(src, os.path.join(obj_dir, os.path.relpath(src, csrc).replace(os.sep, "_") + ".o")) for src in sources(csrc)]
    units.append((DRIVER, os.path.join(obj_dir, "reference_bench.o")))
    jobs = jobs or min(16, os.cpu_count() or 4)
    with concurrent.futures.ThreadPoolExecutor(jobs) as pool:
        futures = [pool.submit(run, [nvcc, *flags, "-c", src, "-o", obj]) for src, obj in units]
        for f in futures:
            f.result()
    run([nvcc, "-o", BINARY, *[obj for _, obj in units], "-lcublas", "-lcudart", "-lpthread",
         "-Xlinker", "-rpath", "-Xlinker", "/usr/local/cuda/lib64", "-Wno-deprecated-gpu-targets"])
    with open(STAMP, "w") as fh:
        fh.write(fingerprint(csrc))
    return BINARY


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--source", default=None, help="checkout of the reference (default: $CUINFER_REFERENCE_SOURCE)")
    parser.add_argument("--jobs", type=int, default=0)
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    print(build(args.source, args.jobs, args.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
