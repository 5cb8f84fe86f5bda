"""Compiles the CUDA sources in this folder into one shared library for sm_100a.

The library is built in-tree (``csrc/_build/``) the first time it is needed and
again whenever a source or a flag changes; a folder that cannot be written falls
back to a per-user folder under the system's temporary directory.  Only ``nvcc``
and the host compiler are needed: no network, no home directory, no Python
extension headers.  While it compiles it prints a line per finished file to
standard error.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libmlxforge_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]
LINK_FLAGS = ["-shared"]


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("MLXFORGE_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("mlxforge_b200: nvcc not found (set CUDA_HOME or MLXFORGE_NVCC); "
                     "the engine has no fallback without its CUDA library")


def source_hash() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + LINK_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"mlxforge_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[mlxforge_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str) -> str:
    cmd = [nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{p.stdout}")
    return src


def library_path(build: bool = True, verbose: Optional[bool] = None) -> str:
    """Path of an up-to-date library, compiling it first if it is stale or absent."""
    d = _build_dir()
    lib = os.path.join(d, LIB_NAME)
    stamp = os.path.join(d, "build.stamp")
    want = source_hash()

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return f.read().strip() == want and os.path.isfile(lib)
        except OSError:
            return False

    if fresh():
        return lib
    if not build:
        raise BuildError(f"mlxforge_b200: {lib} is missing or stale and building was not allowed")
    with open(os.path.join(d, "build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if fresh():
            return lib
        nvcc = find_nvcc()
        srcs = sources()
        t0 = time.time()
        _say(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} into {d} (first call only)")
        objs = {s: os.path.join(d, s[:-3] + ".o") for s in srcs}
        done = 0
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, objs[s]) for s in srcs]
            for fu in as_completed(futs):
                s = fu.result()
                done += 1
                _say(f"  [{done}/{len(srcs)}] {s} ({time.time() - t0:.0f}s)")
        tmp = lib + f".tmp{os.getpid()}"
        cmd = [nvcc] + LINK_FLAGS + ["-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp] + list(objs.values())
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise BuildError(f"link failed:\n{p.stdout}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(want)
        _say(f"done in {time.time() - t0:.0f}s: {lib}")
    return lib


if __name__ == "__main__":
    print(library_path())
